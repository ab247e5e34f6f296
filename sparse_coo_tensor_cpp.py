"""Drop-in for the reference's native extension module of the same name (sparse-extension/setup.py:4-5,
imported at gcn_distr.py:27): `spmm_gpu` and `sparse_coo_tensor_gpu` with the reference's signatures, backed by
the hand-written sm_100a kernels of `cagnet_b200/libcagnet_b200.so` instead of cuSPARSE."""
from cagnet_b200.ops import sparse_coo_tensor_gpu, spmm_gpu  # noqa: F401

__all__ = ["spmm_gpu", "sparse_coo_tensor_gpu"]
