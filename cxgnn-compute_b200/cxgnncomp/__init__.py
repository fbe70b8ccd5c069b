"""Host-side mirror of the `cxgnncomp` Python package of CxGNN-Compute for the aggregation path
(cxgnncomp/__init__.py:1-18 of the reference lists the same names). Operators come from the
`cxgnncomp_backend` module next to this package, which calls the sm_100a library."""
from cxgnncomp_backend import (edge_attention, sage_sum_forward_edge_value, gather, sage_sum_forward, aggr_rel,
                               sage_mean_forward, rel_schedule, target_aggr)

from .schedule import (neighbor_grouping, neighbor_grouping_gpu, partition_2d, reorder_by, remove_from_graph,
                       remove_from_graph_by_edge)
from .partition import partition_2d_gpu, partition_2d_gpu_layered, row_partition_by_nnz, local_rows
from .graph_conv import (MyGATConv, MyGCNConv, MySageConv, MyGINConv, MyRGCNConv, RGCNOP, RGCNOP2, RGCNOP3,
                         RGCNOP_sorted, AggrOP, AggrDirectedOP)
from .graph_kernel import SpMMValOP
from .typed_linear import (TypedLinearE2EOP, TypedLinearS2EOP, TypedLinearS2DMMAggrOP, TypedLinearS2DAggrMMOP,
                           TypedLinearS2DSort, TypedLinearNaiveS2D, TypedLinearS2DPushOP, SelectMMS2EOP)
from .codegen import typed_matmul, spmm_torch, Tuner, compare, prof
from .model import SAGE, GCN, GAT, GIN, RGCN, GNN, get_conv_from_str, get_model_from_str
from .batch import Batch
from .sampler import NeighborSampler
from .neighbor_lstm import NeighborLstmOneByOneOP, NeighborLstmOP, NeighborLstmPadOP
from .train import train_epoch, num_batches
from .timer import TimerOP
from .util import global_tuner
