"""Access to the CUDA library that fails loudly: there is no CPU fallback."""


def require_ext():
    """Returns the ``_C`` binding module or raises RuntimeError if it is not built."""
    try:
        from . import _C
    except ImportError as exc:
        raise RuntimeError(
            "bittorch_b200 requires its CUDA extension to be built "
            f"(python -m bittorch_b200._build): {exc}"
        ) from exc
    return _C


def require_cuda_tensor(t, what: str):
    if not t.is_cuda:
        raise RuntimeError(
            f"bittorch_b200: {what} must be a CUDA tensor — this backend has no CPU path "
            "(use backend='python' on TernaryLinear for the eager reference arithmetic)"
        )
