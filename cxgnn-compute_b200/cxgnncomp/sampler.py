"""Layer-wise neighbour sampling that emits the CSR_Layer batch format the model stacks consume
(cxgnncomp/model.py:55-71 of the reference; the reference takes the batches from its external loader,
cxgnncomp/data_preparation.py:200-230, test/ae/E2_spmm/perf-spmm.py:37-60).

Batch layout: `nodes` lists global ids, seeds first, then the nodes first reached at hop 1, hop 2, ... (each
group in ascending id order). Row r of the batch CSR holds the sampled in-neighbours of nodes[r] as positions
into `nodes`; rows exist for every node that was expanded (all but the last hop's new nodes).
num_node_in_layer = [seeds, after hop 1, ..., after hop L]; num_edge_in_layer[l] = edges of the first
num_node_in_layer[l] rows. Layer i of an L-layer model uses entry L-1-i of both lists."""
import torch

import cxgnncomp_backend

from .batch import Batch


class NeighborSampler:
    """fanouts[h] neighbours per node at hop h+1 counted from the seeds. The draw for a node depends only on
    (seed of the call, node id), so a batch is reproducible from (seeds, seed)."""

    def __init__(self, graph_ptr, graph_idx, fanouts):
        self.ptr, self.idx = graph_ptr, graph_idx
        self.fanouts = [int(f) for f in fanouts]
        self.num_nodes = graph_ptr.shape[0] - 1
        # global id -> position in the batch, -1 outside the batch; cleared after every batch
        self.local_of = torch.full((self.num_nodes,), -1, dtype=torch.int64, device=graph_ptr.device)
        self.n_fresh = torch.zeros(1, dtype=torch.int64, device=graph_ptr.device)
        self._fresh_buf = torch.empty(0, dtype=torch.int64, device=graph_ptr.device)

    def _scratch(self, n):
        if self._fresh_buf.shape[0] < n:
            self._fresh_buf = torch.empty(max(n, 2 * self._fresh_buf.shape[0]), dtype=torch.int64,
                                          device=self._fresh_buf.device)
        return self._fresh_buf

    def sample(self, seeds, seed=0):
        """seeds: distinct int64 global ids on the graph's device. Returns (nodes, ptr, idx, num_node_in_layer,
        num_edge_in_layer) with ptr / idx int64 on the device."""
        dev = seeds.device
        local_of = self.local_of
        nodes = [seeds]
        n_known = seeds.shape[0]
        local_of[seeds] = torch.arange(n_known, device=dev)
        num_node, num_edge = [n_known], []
        frontier = seeds
        ptr_parts, idx_parts, edge_base = [torch.zeros(1, dtype=torch.int64, device=dev)], [], 0
        for hop, fanout in enumerate(self.fanouts):
            out_ptr, picked = cxgnncomp_backend.sample_neighbors(self.ptr, self.idx, frontier, fanout,
                                                                 seed * 1000003 + hop)
            # ids seen for the first time: claimed once each on the device, then sorted so that the batch does
            # not depend on the order in which threads claimed them
            fresh_buf = self._scratch(min(picked.shape[0], self.num_nodes))
            cxgnncomp_backend.renumber_claim(picked, local_of, fresh_buf, self.n_fresh)
            fresh = torch.sort(fresh_buf[:int(self.n_fresh)]).values
            idx_parts.append(cxgnncomp_backend.renumber_assign(fresh, n_known, picked, local_of))
            ptr_parts.append(out_ptr[1:] + edge_base)
            edge_base += picked.shape[0]
            n_known += fresh.shape[0]
            nodes.append(fresh)
            num_node.append(n_known)
            num_edge.append(edge_base)
            frontier = fresh
        nodes = torch.cat(nodes)
        local_of[nodes] = -1
        return nodes, torch.cat(ptr_parts), torch.cat(idx_parts), num_node, num_edge

    def batch(self, x, seeds, seed=0, y=None):
        """A `Batch` with the features (and labels of the seeds) gathered for the sampled nodes."""
        nodes, ptr, idx, num_node, num_edge = self.sample(seeds, seed)
        return Batch(x[nodes], ptr, idx, num_node, num_edge, target=nodes, y=None if y is None else y[seeds])
