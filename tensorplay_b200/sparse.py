"""``sparse``: PyTorch's package, plus the constructors and conversions that the reference also lists here
(tensorplay/sparse/__init__.py) and that PyTorch keeps at its top level or as tensor methods."""
import torch as _torch

# (no star import: PyTorch's ``sparse.__all__`` names a function that the module does not define)
globals().update({_n: getattr(_torch.sparse, _n) for _n in dir(_torch.sparse) if not _n.startswith("_")})


def add(a, b, *, alpha=1):
    return _torch.add(a, b, alpha=alpha)


def mul(a, b):
    return _torch.mul(a, b)


def coalesce(t):
    return t.coalesce()


def sparse_mask(t, mask):
    return t.sparse_mask(mask)


def to_dense(t):
    return t.to_dense()


def to_sparse(t, *args, **kwargs):
    return t.to_sparse(*args, **kwargs)


def to_sparse_csr(t, **kw):
    return t.to_sparse_csr(**kw)


def to_sparse_csc(t, **kw):
    return t.to_sparse_csc(**kw)


def to_sparse_bsr(t, blocksize, **kw):
    return t.to_sparse_bsr(blocksize, **kw)


def to_sparse_bsc(t, blocksize, **kw):
    return t.to_sparse_bsc(blocksize, **kw)


def solve(A, b):
    """Solves ``A x = b`` for a sparse CSR (or any sparse layout) ``A``: PyTorch's sparse solver where this build has
    one, the dense solver otherwise."""
    try:
        return _torch.sparse.spsolve(A if A.layout == _torch.sparse_csr else A.to_sparse_csr(), b)
    except (RuntimeError, NotImplementedError, AttributeError):
        return _torch.linalg.solve(A.to_dense(), b)


def __getattr__(name):
    for ns in (_torch.sparse, _torch):
        try:
            return getattr(ns, name)
        except AttributeError:
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
