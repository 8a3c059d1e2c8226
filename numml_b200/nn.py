"""Graph-convolution layers whose graph argument is a sparse matrix.

Mirror of the reference's ``numml/nn.py`` (layers ``:6-168``, containers and the parameter-vector
helpers ``:171-234``): same class names, constructor arguments, parameter names (``weights``,
``bias``) and arithmetic, so that a ``state_dict`` moves between the two.  The sparse work of a layer
is the SpMM ``A @ X`` (``SparseCSRTensor.__matmul__`` -> ``spdmm``) and, when the layer normalises,
the row sums of A (``SparseCSRTensor.row_sum`` -> ``sprowsum``); both run on this package's CUDA
kernels and are differentiable with respect to the stored values of A as well as X.
"""
import torch


def _as_feature_matrix(X):
    """Node features as [nodes, channels]; a vector is one channel."""
    return X.unsqueeze(1) if X.ndim == 1 else X


def _inv_sqrt_degree(row_sums):
    """Diagonal of D~^(-1/2) for A~ = A + I, as a column that broadcasts over the channels."""
    return ((row_sums + 1.) ** -0.5)[:, None]


class _GraphConv(torch.nn.Module):
    """What the two layers share: channel counts, the normalisation switch, the bias."""

    def __init__(self, in_channels, out_channels, normalize, weight_shape):
        super().__init__()
        # registration order (weights, then bias) fixes the layout of model_to_vector
        self.weights = torch.nn.Parameter(torch.randn(*weight_shape))
        self.bias = torch.nn.Parameter(torch.randn(out_channels))
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.normalize = normalize


class GCNConv(_GraphConv):
    """Kipf & Welling graph convolution on a matrix:
    ``Y = D~^(-1/2) (A + I) D~^(-1/2) X W + b`` (``normalize=True``) or ``Y = A X W + b``.
    Reference ``numml/nn.py:6-101``."""

    def __init__(self, in_channels, out_channels, normalize=True):
        super().__init__(in_channels, out_channels, normalize, (in_channels, out_channels))

    def _convolve(self, matmul, row_sums, X):
        Z = _as_feature_matrix(X) @ self.weights
        if self.normalize:
            d = _inv_sqrt_degree(row_sums())
            Z = d * Z
            out = d * (matmul(Z) + Z)            # (A + I) Z without forming A + I
        else:
            out = matmul(Z)
        return out + self.bias

    def forward(self, A, X):
        """A: ``SparseCSRTensor`` or ``LinearOperator``; X: [nodes, in_channels] or [nodes]."""
        return self._convolve(lambda Z: A @ Z, A.row_sum, X)

    def forward_dense(self, A, X):
        """The same layer evaluated on ``A.to_dense()`` (a check, and the only form that runs on CPU)."""
        Ad = A.to_dense()
        return self._convolve(lambda Z: Ad @ Z, lambda: Ad.sum(dim=1), X)


class TAGConv(_GraphConv):
    """Topology-adaptive graph convolution: ``Y = sum_{j=1..k} P^j(X) W_j + b`` where one hop is
    ``P(X) = A X`` or, normalised, ``P(X) = d * (A (d * X + X))`` with ``d = (rowsum(A) + 1)^(-1/2)``
    (the reference's update, ``numml/nn.py:104-168``, kept as it is written there)."""

    def __init__(self, in_channels, out_channels, k=2, normalize=True):
        super().__init__(in_channels, out_channels, normalize, (k, in_channels, out_channels))
        self.k = k

    def forward(self, A, X):
        Xc = _as_feature_matrix(X)
        d = _inv_sqrt_degree(A.row_sum()) if self.normalize else None
        H = None
        for j in range(self.k):
            Xc = d * (A @ (d * Xc + Xc)) if self.normalize else A @ Xc
            term = Xc @ self.weights[j]
            H = term if H is None else H + term
        if H is None:                                  # k = 0: only the bias
            H = torch.zeros(Xc.shape[0], self.out_channels, dtype=Xc.dtype, device=Xc.device)
        return H + self.bias


class SeqWrapper(torch.nn.Module):
    """Lets a layer that ignores the graph (an activation, a ``Linear``) sit in a ``Sequential``."""

    def __init__(self, module):
        super().__init__()
        self.module = module

    def forward(self, A, x):
        return self.module(x)


class Sequential(torch.nn.Module):
    """Chain of layers called as ``layer(A, X)``; the result is squeezed (reference ``:180-188``)."""

    def __init__(self, *args):
        super().__init__()
        self.modlist = torch.nn.ModuleList(list(args))

    def forward(self, A, X):
        for layer in self.modlist:
            X = layer(A, X)
        return torch.squeeze(X)


def model_to_vector(model):
    """Every tensor of ``model.state_dict()`` flattened into one float32 vector on the host, in
    state-dict order (reference ``numml/nn.py:193-211``)."""
    parts = [t.detach().flatten().to(device='cpu', dtype=torch.float32) for t in model.state_dict().values()]
    return torch.cat(parts) if parts else torch.zeros(0)


def vector_to_model(model, weights_vector):
    """Replace each parameter of ``model`` by a view of its slice of ``weights_vector`` (in
    ``named_parameters`` order), so that a loss computed with the model differentiates with respect
    to the vector (reference ``numml/nn.py:221-234``).  The parameters stop being ``Parameter``s."""
    offset = 0
    for name, p in list(model.named_parameters()):
        owner_path, _, attr = name.rpartition('.')
        owner = model.get_submodule(owner_path) if owner_path else model
        count = p.numel()
        delattr(owner, attr)
        setattr(owner, attr, weights_vector[offset:offset + count].view_as(p))
        offset += count
