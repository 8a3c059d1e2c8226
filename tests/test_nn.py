"""Graph-convolution layers against outputs of the reference's own layers (committed golden vectors,
made by tests/golden/make_golden.py).  The dense evaluation and the container helpers run on CPU;
the sparse evaluation, which goes through the SpMM and row-sum kernels, needs the GPU."""
import pytest
import torch

from parity import assert_close, assert_same, case
import numml_b200.nn as nn
import numml_b200.sparse as sp

LAYERS = {
    "gcn_norm": lambda: nn.GCNConv(4, 3, normalize=True),
    "gcn_plain": lambda: nn.GCNConv(4, 3, normalize=False),
    "tag_norm": lambda: nn.TAGConv(4, 3, k=2, normalize=True),
    "tag_plain": lambda: nn.TAGConv(4, 3, k=3, normalize=False),
}
TOL = 1e-5     # float32, norm-wise; dense products are summed in another order than on the reference's CPU


def _setup(golden_api, tag, device):
    g = case(golden_api, "gnn")
    layer = LAYERS[tag]()
    with torch.no_grad():
        layer.weights.copy_(g[f"{tag}/weights"])
        layer.bias.copy_(g[f"{tag}/bias"])
    layer = layer.to(device)
    A = sp.SparseCSRTensor((g["A_data"].clone(), g["A_indices"], g["A_indptr"]), (30, 30)).to(device)
    A.requires_grad = True
    X = g["X"].clone().to(device).requires_grad_(True)
    return g, layer, A, X


@pytest.mark.parametrize("tag", ["gcn_norm", "gcn_plain"])
def test_dense_evaluation_matches_reference_layer(golden_api, tag):
    g, layer, A, X = _setup(golden_api, tag, "cpu")
    Y = layer.forward_dense(A, X)
    assert_close(g[f"{tag}/Y"], Y.detach(), "Y", TOL)


def test_parameter_vector_round_trip():
    torch.manual_seed(0)
    model = nn.Sequential(nn.GCNConv(4, 3), nn.SeqWrapper(torch.nn.Tanh()), nn.TAGConv(3, 1, k=2))
    v = nn.model_to_vector(model)
    assert v.dtype == torch.float32 and v.numel() == 4 * 3 + 3 + 2 * 3 * 1 + 1
    assert torch.equal(v[:12].view(4, 3), model.modlist[0].weights.detach())     # weights before bias
    w = (v * 2).requires_grad_(True)
    nn.vector_to_model(model, w)
    assert torch.equal(model.modlist[0].weights, (w[:12]).view(4, 3))
    assert not isinstance(model.modlist[0].weights, torch.nn.Parameter)
    model.modlist[2].bias.sum().backward()                                       # gradient reaches the vector
    assert w.grad[-1] == 1 and w.grad[:-1].abs().sum() == 0
    A = sp.eye(5)
    out = model.modlist[1](A, torch.ones(5, 3))                                  # wrapper ignores the graph
    assert torch.allclose(out, torch.tanh(torch.ones(5, 3)))


@pytest.mark.gpu
@pytest.mark.parametrize("tag", sorted(LAYERS))
def test_layers_match_reference_on_gpu(golden_api, tag):
    g, layer, A, X = _setup(golden_api, tag, "cuda")
    Y = layer(A, X)
    assert_close(g[f"{tag}/Y"], Y.detach().cpu(), "Y", TOL)
    (Y * g[f"{tag}/w"].cuda()).sum().backward()
    assert_close(g[f"{tag}/grad_weights"], layer.weights.grad.cpu(), "grad weights", TOL)
    assert_close(g[f"{tag}/grad_bias"], layer.bias.grad.cpu(), "grad bias", TOL)
    assert_close(g[f"{tag}/grad_A"], A.data.grad.cpu(), "grad A", TOL)
    assert_close(g[f"{tag}/grad_X"], X.grad.cpu(), "grad X", TOL)


@pytest.mark.gpu
def test_row_sum_is_the_reference_sum_bit_for_bit(golden_api):
    g = case(golden_api, "gnn")
    A = sp.SparseCSRTensor((g["A_data"].clone(), g["A_indices"], g["A_indptr"]), (30, 30)).to("cuda")
    A.requires_grad = True
    s = A.row_sum()
    assert_same(case(golden_api, "rowsum")["values"], s.detach().cpu(), "row sums")
    up = torch.arange(1, 31, dtype=torch.float32, device="cuda")
    (s * up).sum().backward()
    counts = (g["A_indptr"][1:] - g["A_indptr"][:-1])
    assert torch.equal(A.data.grad.cpu(), torch.repeat_interleave(up.cpu(), counts))


@pytest.mark.gpu
def test_sequential_runs_on_gpu(golden_api):
    g = case(golden_api, "gnn")
    torch.manual_seed(1)
    model = nn.Sequential(nn.GCNConv(4, 8), nn.SeqWrapper(torch.nn.ReLU()), nn.TAGConv(8, 1, k=2)).cuda()
    A = sp.SparseCSRTensor((g["A_data"].clone(), g["A_indices"], g["A_indptr"]), (30, 30)).to("cuda")
    A.requires_grad = True
    y = model(A, g["X"].cuda())
    assert y.shape == (30,)
    y.square().sum().backward()
    assert A.data.grad is not None and torch.isfinite(A.data.grad).all()
    dense = model.modlist[0].forward_dense(A, g["X"].cuda())
    assert_close(dense.detach().cpu(), model.modlist[0](A, g["X"].cuda()).detach().cpu(), "sparse vs dense", TOL)
