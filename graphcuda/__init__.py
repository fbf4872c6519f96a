"""Drop-in alias: ``import graphcuda`` resolves to the B200 engine with the
reference's public names (src/graphcuda/__init__.py:20-28)."""
from graphcuda_b200 import (GCNConv, gemm_cublas, matmul1, matmul2, matmul3, matmul4,  # noqa: F401
                            spmm_cusparse)
from graphcuda_b200 import _graphcuda  # noqa: F401

__all__ = ["GCNConv", "matmul1", "matmul2", "matmul3", "matmul4", "gemm_cublas", "spmm_cusparse"]
