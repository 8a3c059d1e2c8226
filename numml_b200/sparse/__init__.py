from ._csr import *  # noqa: F401,F403
from ._csr import SparseCSRTensor, coo_to_csr, eye, diag, spouter, spgemv, spgemm, spdmm, sptranspose  # noqa: F401
from ._linear_operator import LinearOperator  # noqa: F401
from . import linalg  # noqa: F401
