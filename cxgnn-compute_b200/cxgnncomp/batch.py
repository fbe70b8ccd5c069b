"""Batch container in the CSR_Layer format (cxgnncomp/batch.py:7-91 of the reference, without its dgl import) and
the on-disk cache of partitioned graphs.

Nodes are ordered so that the destinations of layer l are a prefix of the nodes of layer l+1; one `ptr` / `idx`
pair serves every layer: layer i of an L-layer model uses the first num_node_in_layer[L-1-i] rows and the first
num_edge_in_layer[L-1-i] edges (cxgnncomp/model.py:55-71).

Wire format (batch.py:38-62 of the reference): one directory per sub-graph with raw little-endian dumps
`x.dat` (float32), `ptr.dat`, `idx.dat`, `target.dat` (int64), each present only when the field is set. The
multi-GPU script names the directories `.cache/{dataset}_{num_device}_{rank}_{layer}_{src_rank}` and keeps the
layer sizes in `.cache/{dataset}_num_node_in_layer.txt`, one integer per line
(test/1-kernels/test_mgpu_model.py:548-570); `cache_dir`, `save_num_node_in_layer` and `load_num_node_in_layer`
reproduce that naming."""
import os

import numpy as np
import torch


class Batch:

    def __init__(self, x, ptr, idx, num_node_in_layer=None, num_edge_in_layer=None, target=None, edge_index=None,
                 y=None):
        self.x, self.ptr, self.idx = x, ptr, idx
        self.num_node_in_layer = num_node_in_layer
        self.num_edge_in_layer = num_edge_in_layer
        self.target = target
        self.edge_index = edge_index
        self.y = y

    def to(self, device):
        for name in ("x", "ptr", "idx", "target", "y", "edge_index"):
            t = getattr(self, name)
            if isinstance(t, torch.Tensor):
                setattr(self, name, t.to(device))
        return self

    def totype(self, dtype):
        """Index arrays to `dtype` (batch.py:85-88)."""
        self.ptr = self.ptr.to(dtype)
        self.idx = self.idx.to(dtype)
        if self.target is not None:
            self.target = self.target.to(dtype)

    def tofile(self, directory):
        """Writes the set fields as raw arrays, byte for byte what the reference writes: the tensor's own dtype
        and layout (`tensor.cpu().numpy().tofile`), so float32 features and int64 indices give the documented
        format. The directory is created when missing."""
        os.makedirs(directory, exist_ok=True)
        for name in ("x", "ptr", "idx", "target"):
            t = getattr(self, name)
            if t is not None:
                t.detach().cpu().contiguous().numpy().tofile(os.path.join(directory, name + ".dat"))

    def fromfile(self, directory, feat_len=None):
        """Reads back what `tofile` wrote into this object (instance method, like the reference's): x as float32
        (flat, as the reference leaves it, or [-1, feat_len] when feat_len is given), ptr / idx / target as int64;
        fields whose file is missing keep their value. Returns self."""
        def path(name):
            return os.path.join(directory, name + ".dat")

        if os.path.exists(path("x")):
            self.x = torch.from_numpy(np.fromfile(path("x"), dtype=np.float32))
            if feat_len:
                self.x = self.x.view(-1, feat_len)
        if os.path.exists(path("ptr")):
            self.ptr = torch.from_numpy(np.fromfile(path("ptr"), dtype=np.int64))
        else:
            print(path("ptr"), "not found")
        if os.path.exists(path("idx")):
            self.idx = torch.from_numpy(np.fromfile(path("idx"), dtype=np.int64))
        if os.path.exists(path("target")):
            self.target = torch.from_numpy(np.fromfile(path("target"), dtype=np.int64))
        return self


def cache_dir(root, dataset, num_device, rank, layer, src_rank):
    """Directory of sub-graph (rank <- src_rank) of `layer` in a partition cache
    (test/1-kernels/test_mgpu_model.py:552: f".cache/{dataset}_{num_device}_{rank}_{l}_{it}")."""
    return os.path.join(root, f"{dataset}_{num_device}_{rank}_{layer}_{src_rank}")


def save_num_node_in_layer(root, dataset, num_node_in_layer):
    """One integer per line into {root}/{dataset}_num_node_in_layer.txt (test_mgpu_model.py:556-558)."""
    os.makedirs(root, exist_ok=True)
    with open(os.path.join(root, f"{dataset}_num_node_in_layer.txt"), "w") as f:
        for item in num_node_in_layer:
            print(int(item), file=f)


def load_num_node_in_layer(root, dataset):
    with open(os.path.join(root, f"{dataset}_num_node_in_layer.txt")) as f:
        return [int(line) for line in f if line.strip()]


def save_partition_cache(root, dataset, num_device, rank, graphs_in_layer, num_node_in_layer=None):
    """graphs_in_layer[l][i] = Batch(ptr, idx, target) of (this rank <- source rank i) in layer l, as
    partition_2d_gpu_layered produces them; one directory each, in the reference's naming."""
    for layer, graphs in enumerate(graphs_in_layer):
        for src_rank, g in enumerate(graphs):
            g.tofile(cache_dir(root, dataset, num_device, rank, layer, src_rank))
    if num_node_in_layer is not None:
        save_num_node_in_layer(root, dataset, num_node_in_layer)


def load_partition_cache(root, dataset, num_device, rank, num_layer, skip_input=False):
    """Inverse of save_partition_cache (test_mgpu_model.py:561-570); with skip_input layer 0 stays empty."""
    graphs_in_layer = [[] for _ in range(num_layer)]
    for layer in range(num_layer):
        if skip_input and layer == 0:
            continue
        for src_rank in range(num_device):
            b = Batch(x=None, ptr=None, idx=None, target=None)
            b.fromfile(cache_dir(root, dataset, num_device, rank, layer, src_rank))
            graphs_in_layer[layer].append(b)
    return graphs_in_layer
