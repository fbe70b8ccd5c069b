"""Model stacks over the CSR_Layer format: the `forward_cxg` branches of the reference's model zoo
(cxgnncomp/model.py:55-71,166-191,251-273) without its DGL / PyG branches."""
import torch
import torch.nn.functional as F

from .graph_conv import MyGATConv, MyGCNConv, MyGINConv, MyRGCNConv, MySageConv


def get_conv_from_str(name, in_channels, out_channels, num_heads=1, num_rel=1, concat=False):
    name = name.upper()
    if name == "SAGE":
        return MySageConv(in_channels, out_channels)
    if name == "GCN":
        return MyGCNConv(in_channels, out_channels)
    if name == "GIN":
        return MyGINConv(in_channels, out_channels)
    if name == "GAT":
        return MyGATConv(in_channels, out_channels, heads=num_heads, concat=concat)
    if name == "RGCN":
        return MyRGCNConv(in_channels, out_channels, num_rel)
    raise ValueError(f"unknown model {name}")


class GNN(torch.nn.Module):
    """conv -> BatchNorm -> ReLU -> dropout per hidden layer, log_softmax at the end (model.py:17-71)."""

    def __init__(self, conv, in_channels, hidden_channels, out_channels, num_layers, dropout=0.5, num_heads=1,
                 num_rel=1):
        super().__init__()
        self.conv_name = conv.upper()
        self.num_layers = num_layers
        self.dropout = dropout
        self.num_rel = num_rel
        dims = [in_channels] + [hidden_channels] * (num_layers - 1) + [out_channels]
        self.convs = torch.nn.ModuleList()
        self.bns = torch.nn.ModuleList()
        for i in range(num_layers):
            concat = self.conv_name == "GAT" and i < num_layers - 1
            width = dims[i + 1] // num_heads if concat else dims[i + 1]
            self.convs.append(get_conv_from_str(conv, dims[i], width, num_heads, num_rel, concat))
            if i < num_layers - 1:
                self.bns.append(torch.nn.BatchNorm1d(dims[i + 1]))

    def reset_parameters(self):
        for c in self.convs:
            c.reset_parameters()
        for b in self.bns:
            b.reset_parameters()

    def forward(self, batch, edge_types=None):
        return self.forward_cxg(batch, edge_types)

    def forward_cxg(self, batch, edge_types=None):
        x = batch.x
        L = self.num_layers
        for i, conv in enumerate(self.convs):
            num_node = int(batch.num_node_in_layer[L - 1 - i])
            num_edge = int(batch.num_edge_in_layer[L - 1 - i]) if batch.num_edge_in_layer is not None else batch.idx.shape[0]
            if self.conv_name == "GAT":
                x = conv(x, batch.ptr, batch.idx, num_node, int(batch.num_node_in_layer[L - i]), num_edge)
            elif self.conv_name == "RGCN":
                x = conv(x, batch.ptr[:num_node + 1], batch.idx[:num_edge], edge_types[:num_edge], num_node)
            else:
                x = conv(x, batch.ptr[:num_node + 1], batch.idx[:num_edge], num_node)
            if i != L - 1:
                x = F.dropout(F.relu(self.bns[i](x)), p=self.dropout, training=self.training)
        return x.log_softmax(dim=-1)


def SAGE(in_c, hid, out_c, num_layers, dropout=0.5):
    return GNN("SAGE", in_c, hid, out_c, num_layers, dropout)


def GCN(in_c, hid, out_c, num_layers, dropout=0.5):
    return GNN("GCN", in_c, hid, out_c, num_layers, dropout)


def GIN(in_c, hid, out_c, num_layers, dropout=0.5):
    return GNN("GIN", in_c, hid, out_c, num_layers, dropout)


def GAT(in_c, hid, out_c, num_layers, heads=4, dropout=0.5):
    return GNN("GAT", in_c, hid, out_c, num_layers, dropout, num_heads=heads)


def RGCN(in_c, hid, out_c, num_layers, num_rel, dropout=0.5):
    return GNN("RGCN", in_c, hid, out_c, num_layers, dropout, num_rel=num_rel)


def get_model_from_str(name, in_c, hid, out_c, num_layers, num_heads=1, num_rel=1, dropout=0.5):
    return GNN(name, in_c, hid, out_c, num_layers, dropout, num_heads=num_heads, num_rel=num_rel)
