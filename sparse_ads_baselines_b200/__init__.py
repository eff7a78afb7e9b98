"""B200-native table-batched embedding bags (TBE).

The package is a drop-in for the TBE hot path of sparse-ads-baselines: it ships modules with the
reference's own names (``table_batched_embeddings`` -- the extension functions --,
``table_batched_embeddings_ops``, ``sparse_embedding_cuda``, ``sparse_embedding_cuda_ops``) on top
of ``libtbe_b200.so``, a C-ABI CUDA library for sm_100a declared in ``include/tbe_b200.h``.

``install_reference_names()`` registers those modules under their bare reference names in
``sys.modules`` so code written as ``import table_batched_embeddings_ops`` runs unchanged.
"""
import importlib
import sys

__all__ = ["install_reference_names"]

_REFERENCE_MODULES = (
    "table_batched_embeddings",
    "table_batched_embeddings_ops",
    "sparse_embedding_cuda",
    "sparse_embedding_cuda_ops",
)


def install_reference_names():
    """Makes ``import table_batched_embeddings_ops`` (etc.) resolve to this package's modules."""
    for name in _REFERENCE_MODULES:
        try:
            mod = importlib.import_module(__name__ + "." + name)
        except ModuleNotFoundError as e:  # a module of this package that is not built yet
            if e.name != __name__ + "." + name:
                raise
            continue
        sys.modules.setdefault(name, mod)
