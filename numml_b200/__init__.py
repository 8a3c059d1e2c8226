"""numml_b200: the differentiable CSR hot path of numml (SpMV / SpMM / SpGEMM / triangular solve,
forward and backward) as hand-written sm_100a CUDA kernels behind numml's own sparse API.

    import numml_b200.sparse as sp
    A = sp.SparseCSRTensor((data, indices, indptr), shape).to('cuda')
    y = A @ x
"""
__version__ = "0.1.0"
