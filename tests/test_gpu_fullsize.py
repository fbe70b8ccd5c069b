"""Configuration 5 at full size (111 M nodes, 1.6 G edges, F = 128 bf16, int32 column ids) on one GPU, checked
through properties that do not need a second full pass on the CPU: a checksum of checksums (column sums), the
C oracle on sampled rows, exact float64 sums of the heaviest rows, and bit-identical repetition."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def test_config5_full_size_properties(cuda):
    import cxgnncomp_backend as be
    from cxgnncomp import synthetic
    if torch.cuda.get_device_properties(0).total_memory < 150e9:
        pytest.skip("needs a 180 GB device")
    dev = torch.device("cuda")
    n, e_und = synthetic.CONFIG_SHAPES["papers_like"]
    ptr, idx = synthetic.powerlaw_graph(n, e_und, seed=0, device=dev, idx_dtype=torch.int32)
    nnz = idx.shape[0]
    assert nnz == 2 * e_und + n
    x = synthetic.node_features(n, 128, seed=0, device=dev, dtype=torch.bfloat16)
    y = be.run_spmm_configurable(ptr, idx, x, n)
    y2 = be.run_spmm_configurable(ptr, idx, x, n)
    assert torch.equal(y, y2)  # no atomics, no dependence on scheduling
    del y2

    # checksum of checksums: sum_r y[r, :] = sum_s (number of edges that read s) * x[s, :]
    count = torch.zeros(n, dtype=torch.int64, device=dev)
    for e0 in range(0, nnz, 1 << 28):
        count += torch.bincount(idx[e0:e0 + (1 << 28)], minlength=n)
    assert int(count.sum()) == nnz
    want = torch.zeros(128, dtype=torch.float64, device=dev)
    got = torch.zeros(128, dtype=torch.float64, device=dev)
    energy = torch.zeros((), dtype=torch.float64, device=dev)
    for r0 in range(0, n, 1 << 22):
        r1 = min(n, r0 + (1 << 22))
        want += (x[r0:r1].double() * count[r0:r1, None].double()).sum(0)
        yd = y[r0:r1].double()
        got += yd.sum(0)
        energy += (yd * yd).sum()
    # every output carries one bf16 rounding (2^-9 relative, random sign): the column sums differ from the exact
    # ones by about 2^-9 * sqrt(sum y^2) / sqrt(3) ~ 20; allow ten times that
    noise = float(energy.sqrt()) * 2.0 ** -9
    assert float((got - want).abs().max()) < 6 * noise
    assert float((got - want).abs().max()) < 1e-3 * float(want.abs().max())
    del count

    # sampled rows against the C restatement of the reference's sequential sum (rows of up to 50,000 edges)
    deg = ptr[1:] - ptr[:-1]
    g = torch.Generator(device=dev).manual_seed(3)
    rows = torch.randint(0, n, (3000,), device=dev, generator=g)
    rows = rows[deg[rows] <= 50_000].unique()
    sub_ptr = torch.zeros(rows.shape[0] + 1, dtype=torch.int64, device=dev)
    torch.cumsum(deg[rows], 0, out=sub_ptr[1:])
    pos = torch.arange(int(sub_ptr[-1]), device=dev) - torch.repeat_interleave(sub_ptr[:-1], deg[rows]) + \
        torch.repeat_interleave(ptr[rows], deg[rows])
    cols = idx[pos].long()
    uniq, inv = torch.unique(cols, return_inverse=True)
    ref = oracle.spmm_f64(sub_ptr.cpu(), inv.cpu(), x[uniq].cpu())
    diff = (y[rows].cpu().double() - ref).abs().amax(1) / ref.abs().amax(1).clamp(min=1e-30)
    assert float(diff.max()) < 1e-2  # one bf16 rounding of an fp32 sum

    # the five heaviest rows (tens of millions of edges each) against float64 sums on the device
    for r in torch.topk(deg, 5).indices.tolist():
        e0, e1 = int(ptr[r]), int(ptr[r + 1])
        acc = torch.zeros(128, dtype=torch.float64, device=dev)
        for c0 in range(e0, e1, 1 << 22):
            acc += x[idx[c0:min(e1, c0 + (1 << 22))].long()].double().sum(0)
        assert float((y[r].double() - acc).abs().max()) < 1e-2 * float(acc.abs().max())
