"""Neighbour sampler and the mini-batch step in the CSR_Layer format (configuration 3 in small)."""
import pytest
import torch

import oracle
from helpers import random_csr, randn, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fanout", [1, 5, 15, 64])
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_sample_neighbors_bit_exact(cuda, fanout, idx_dtype):
    """Bit-exact against the C restatement, and the properties of a draw without replacement."""
    import cxgnncomp_backend as be
    ptr, idx = random_csr(400, 400, 12, seed=80, hub=900)
    frontier = torch.randperm(400, generator=torch.Generator().manual_seed(81))[:250]
    out_ptr, out = be.sample_neighbors(ptr.cuda(), idx.to(idx_dtype).cuda(), frontier.cuda(), fanout, seed=7)
    want_ptr, want = oracle.sample_neighbors(ptr, idx, frontier, fanout, 7)
    assert torch.equal(out_ptr.cpu(), want_ptr) and torch.equal(out.cpu(), want)
    deg = ptr[frontier + 1] - ptr[frontier]
    assert torch.equal(out_ptr.cpu()[1:] - out_ptr.cpu()[:-1], deg.clamp(max=fanout))
    # every sampled row is a sub-multiset of the node's full row, in the row's order
    for i in (0, 17, 100, 249):
        row = idx[ptr[frontier[i]]:ptr[frontier[i] + 1]].tolist()
        got = out.cpu()[out_ptr[i]:out_ptr[i + 1]].tolist()
        it = iter(row)
        assert all(any(g == r for r in it) for g in got)
    # another seed draws another sample for the rows that are cut
    _, out2 = be.sample_neighbors(ptr.cuda(), idx.cuda(), frontier.cuda(), fanout, seed=8)
    if fanout < 12:
        assert not torch.equal(out2.cpu(), want)


def test_sampling_is_uniform(cuda):
    """A node of degree 40 sampled 5 at a time over 4000 seeds: every neighbour position is drawn with
    frequency 1/8 within 4 standard deviations."""
    import cxgnncomp_backend as be
    ptr = torch.tensor([0, 40])
    idx = torch.arange(40)
    counts = torch.zeros(40)
    f = torch.zeros(1, dtype=torch.int64).cuda()
    for s in range(4000):
        _, out = be.sample_neighbors(ptr.cuda(), idx.cuda(), f, 5, seed=s)
        counts[out.cpu()] += 1
    sd = (4000 * 0.125 * 0.875) ** 0.5
    assert float((counts - 500).abs().max()) < 4 * sd


def test_batch_format_and_training_step(cuda):
    """The sampler's batch obeys the prefix layout; a 3-layer SAGE forward / backward over it equals the torch
    index_add formulation on the CPU with the same weights; an optimizer step lowers the loss."""
    import cxgnncomp
    torch.manual_seed(5)
    n, classes = 3000, 7
    ptr, idx = random_csr(n, n, 14, seed=90, hub=500, empty_frac=0.02)
    x = randn((n, 20), 91)
    y = torch.randint(0, classes, (n,), generator=torch.Generator().manual_seed(92))
    sampler = cxgnncomp.NeighborSampler(ptr.cuda(), idx.cuda(), [6, 4, 3])
    seeds = torch.randperm(n, generator=torch.Generator().manual_seed(93))[:64].cuda()
    nodes, bptr, bidx, num_node, num_edge = sampler.sample(seeds, seed=3)
    assert torch.equal(nodes[:64], seeds) and len(num_node) == 4 and len(num_edge) == 3
    assert nodes.unique().shape[0] == nodes.shape[0] == num_node[3]
    assert bptr.shape[0] == num_node[2] + 1 and int(bptr[-1]) == bidx.shape[0] == num_edge[2]
    for l in range(3):
        assert int(bptr[num_node[l]]) == num_edge[l]
        assert int(bidx[:num_edge[l]].max()) < num_node[l + 1]  # sources of layer l lie in the next prefix
    # rows are true neighbours: global ids of a few rows
    nc, pc, ic = nodes.cpu(), bptr.cpu(), bidx.cpu()
    for r in (0, 63, 64, num_node[2] - 1):
        full = set(idx[ptr[nc[r]]:ptr[nc[r] + 1]].tolist())
        assert set(nc[ic[pc[r]:pc[r + 1]]].tolist()) <= full
    assert bool((sampler.local_of == -1).all())  # the lookup table is clean again

    model = cxgnncomp.SAGE(20, 32, classes, 3, dropout=0.0).cuda()
    batch = sampler.batch(x.cuda(), seeds, seed=3, y=y.cuda())
    out = model(batch)
    loss = torch.nn.functional.nll_loss(out, batch.y)
    loss.backward()

    # the same network with the aggregation written as index_add on the CPU
    def cpu_forward(params):
        h = x[nc]
        L = 3
        for i in range(L):
            nn_, ne_ = num_node[L - 1 - i], num_edge[L - 1 - i]
            wl, bl, wr = params[f"convs.{i}.lin_l.weight"], params[f"convs.{i}.lin_l.bias"], params[f"convs.{i}.lin_r.weight"]
            if wl.shape[1] > wl.shape[0]:  # wide input: transform, then aggregate (graph_conv.py:142-152)
                agg = oracle.torch_spmm_index_add(h @ wl.t() + bl, pc[:nn_ + 1], ic[:ne_], nn_, mean=True)
            else:
                agg = oracle.torch_spmm_index_add(h, pc[:nn_ + 1], ic[:ne_], nn_, mean=True) @ wl.t() + bl
            h = agg + h[:nn_] @ wr.t()
            if i != L - 1:
                bn_w, bn_b = params[f"bns.{i}.weight"], params[f"bns.{i}.bias"]
                mu, var = h.mean(0), h.var(0, unbiased=False)
                h = torch.relu((h - mu) / torch.sqrt(var + 1e-5) * bn_w + bn_b)
        return h.log_softmax(-1)

    params = {k: v.detach().cpu().clone().requires_grad_(True) for k, v in model.named_parameters()}
    ref = cpu_forward(params)
    assert rel_err(out.detach().cpu(), ref.detach()) < 1e-4
    ref_loss = torch.nn.functional.nll_loss(ref, y[seeds.cpu()])
    ref_loss.backward()
    for k, v in model.named_parameters():
        # (a bias in front of a BatchNorm has a zero gradient: absolute floor)
        diff = float((v.grad.cpu() - params[k].grad).abs().max())
        assert diff < 2e-3 * float(params[k].grad.abs().max()) + 1e-6, k

    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    train = torch.arange(n).cuda()
    first = cxgnncomp.train_epoch(model, opt, sampler, x.cuda(), y.cuda(), train, 256, epoch=0)
    for e in range(1, 6):
        last = cxgnncomp.train_epoch(model, opt, sampler, x.cuda(), y.cuda(), train, 256, epoch=e)
    assert first.shape[0] == cxgnncomp.num_batches(n, 256)
    assert float(last.mean()) < float(first.mean())
    # sampling ahead (a producer thread on a side stream, the default; or the next batch from the training thread)
    # changes neither the batches nor the losses: fresh, identically seeded models, one epoch each
    runs = []
    for prefetch in (True, "stream", False):
        torch.manual_seed(11)
        m2 = cxgnncomp.SAGE(20, 32, classes, 3, dropout=0.0).cuda()
        o2 = torch.optim.Adam(m2.parameters(), lr=0.01)
        runs.append(cxgnncomp.train_epoch(m2, o2, sampler, x.cuda(), y.cuda(), train, 256, epoch=3, prefetch=prefetch))
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])
    # a host-side error inside the producer thread (no feature matrix to index) reaches the caller
    with pytest.raises(TypeError):
        cxgnncomp.train_epoch(m2, o2, sampler, None, y.cuda(), train, 256, epoch=4)
