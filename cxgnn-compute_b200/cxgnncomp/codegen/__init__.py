"""Stand-ins for cxgnncomp/codegen of the reference: the typed matmul entry point (tensor-core kernel
of the library instead of the Triton code generator), the pure-torch SpMM used for validation, and a
Tuner that keeps the reference's interface but has nothing to search."""
from .typed_matmul import typed_matmul
from .torch_spmm import spmm_torch
from .gen_mapping import Tuner
from .util import compare, prof
