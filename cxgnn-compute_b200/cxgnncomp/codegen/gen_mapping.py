class Tuner:
    """The reference's Tuner searches nine launch parameters per (rows, edges, width) by timing trial
    launches and caches the winner (cxgnncomp/codegen/gen_mapping.py:70-176). The kernels here choose
    their schedule from the row width and the edge count, so there is nothing to search: tune_graph
    calls the operator once with placeholder parameters, which the operator ignores."""

    def __init__(self, lazy=True):
        self.lazy = lazy

    def tune_graph(self, num_node, num_edge, feat_len, func, run_param, patience=-1, verbose=False,
                   num_head=1, rettime=False, verbose_all=False):
        out = func(*run_param, 1, 1, 32, 8, 8, feat_len, 32, 0, 0)
        if rettime:
            return out, 0.0
        return out

    def save(self):
        pass
