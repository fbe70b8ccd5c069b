import torch


def spmm_torch(x, ptr, idx, num_nodes, val=None):
    """torch.sparse.mm on a CSR tensor: the formulation the reference validates its kernels against
    (cxgnncomp/codegen/torch_spmm.py:4-9). Runs wherever its inputs live."""
    if val is None:
        val = torch.ones(idx.shape[0], dtype=torch.float32, device=idx.device)
    mat = torch.sparse_csr_tensor(ptr, idx, val, size=(ptr.shape[0] - 1, x.shape[0]), device=ptr.device)
    return torch.sparse.mm(mat, x)
