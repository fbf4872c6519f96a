"""B200-native GCN layer engine with the API of GraphCUDA
(src/graphcuda/__init__.py:20-28 of the reference): ``GCNConv`` plus the
operator functions ``matmul1..4``, ``gemm_cublas``, ``spmm_cusparse``.

Importing the package needs the built C-ABI library
(``python -m graphcuda_b200.build``); there is no fallback path.
"""
import sys as _sys

from . import _lib

# Fail loudly at import when the CUDA library is missing or stale -- except
# while `python -m graphcuda_b200.build` is (re)building it.
if "graphcuda_b200.build" not in getattr(_sys, "orig_argv", []):
    _lib.lib()

from . import _graphcuda  # noqa: E402
from ._graphcuda import (gemm_cublas, matmul1, matmul2, matmul3, matmul4,  # noqa: E402
                         spmm_cusparse)
from .adjacency import (CSRAdjacency, DenseAdjacency, as_adjacency, degree_order, gcn_norm,  # noqa: E402
                        normalized_adjacency)
from .gcn import GCNConv, GCNConvFunction  # noqa: E402
from .feed import PinnedFeed  # noqa: E402
from .graphed import GraphedTrainStep  # noqa: E402
from .losses import argmax_accuracy, log_softmax_nll_loss  # noqa: E402
from .optim import FusedAdam, FusedSGD  # noqa: E402
from .ops import gemm, get_default_precision, set_default_precision  # noqa: E402

cpp_ext = _graphcuda

__all__ = ["GCNConv", "matmul1", "matmul2", "matmul3", "matmul4", "gemm_cublas", "spmm_cusparse"]
