class LinearOperator(object):
    """Wraps callables computing ``A @ x`` (``rm``) and/or ``x @ A`` (``lm``) so that they can
    stand in for a matrix, e.g. as the identity preconditioner of the Krylov solvers
    (reference ``numml/sparse/_linear_operator.py:1-25``)."""

    def __init__(self, shape, rm=None, lm=None):
        self.shape = shape
        self.right_multiply = rm
        self.left_multiply = lm

    def __matmul__(self, x):
        return self.right_multiply(x)

    def __rmatmul__(self, x):
        return self.left_multiply(x)
