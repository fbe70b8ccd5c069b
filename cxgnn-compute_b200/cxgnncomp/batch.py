"""Batch container in the CSR_Layer format (cxgnncomp/batch.py:7-91 of the reference, without its dgl import).

Nodes are ordered so that the destinations of layer l are a prefix of the nodes of layer l+1; one `ptr` / `idx`
pair serves every layer: layer i of an L-layer model uses the first num_node_in_layer[L-1-i] rows and the first
num_edge_in_layer[L-1-i] edges (cxgnncomp/model.py:55-71)."""
import os

import numpy as np
import torch


class Batch:

    def __init__(self, x, ptr, idx, num_node_in_layer, num_edge_in_layer=None, target=None, y=None):
        self.x, self.ptr, self.idx = x, ptr, idx
        self.num_node_in_layer = num_node_in_layer
        self.num_edge_in_layer = num_edge_in_layer
        self.target = target
        self.y = y

    def to(self, device):
        for name in ("x", "ptr", "idx", "target", "y"):
            t = getattr(self, name)
            if isinstance(t, torch.Tensor):
                setattr(self, name, t.to(device))
        return self

    def tofile(self, directory):
        """Raw little-endian dumps x.dat (float32), ptr.dat / idx.dat / target.dat (int64), the wire format of the
        reference's partition cache (batch.py:38-62)."""
        os.makedirs(directory, exist_ok=True)
        self.x.detach().cpu().float().numpy().tofile(os.path.join(directory, "x.dat"))
        self.ptr.cpu().numpy().astype(np.int64).tofile(os.path.join(directory, "ptr.dat"))
        self.idx.cpu().numpy().astype(np.int64).tofile(os.path.join(directory, "idx.dat"))
        if self.target is not None:
            self.target.cpu().numpy().astype(np.int64).tofile(os.path.join(directory, "target.dat"))

    @staticmethod
    def fromfile(directory, feat_len, num_node_in_layer, num_edge_in_layer=None):
        x = torch.from_numpy(np.fromfile(os.path.join(directory, "x.dat"), dtype=np.float32)).view(-1, feat_len)
        ptr = torch.from_numpy(np.fromfile(os.path.join(directory, "ptr.dat"), dtype=np.int64))
        idx = torch.from_numpy(np.fromfile(os.path.join(directory, "idx.dat"), dtype=np.int64))
        tpath = os.path.join(directory, "target.dat")
        target = torch.from_numpy(np.fromfile(tpath, dtype=np.int64)) if os.path.exists(tpath) else None
        return Batch(x, ptr, idx, num_node_in_layer, num_edge_in_layer, target)
