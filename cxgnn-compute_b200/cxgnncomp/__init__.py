"""Host-side mirror of the `cxgnncomp` Python package of CxGNN-Compute for the aggregation path
(cxgnncomp/__init__.py:1-18 of the reference lists the same names). Operators come from the
`cxgnncomp_backend` module next to this package, which calls the sm_100a library."""
from .schedule import (neighbor_grouping, neighbor_grouping_gpu, partition_2d, reorder_by, remove_from_graph,
                       remove_from_graph_by_edge)
from .partition import partition_2d_gpu, partition_2d_gpu_layered, row_partition_by_nnz, local_rows
