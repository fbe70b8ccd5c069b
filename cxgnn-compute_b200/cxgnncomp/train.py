"""Mini-batch epoch loop over sampled CSR_Layer batches: sample -> gather features -> forward -> NLL loss on the
seeds -> backward -> optimizer step (the reference's Trainer.cxg_train_epoch, cxgnncomp/trainer.py:140-175, with
the sampler of this package in place of its external loader)."""
import math

import torch
import torch.nn.functional as F


def num_batches(num_train, batch_size):
    return math.ceil(num_train / batch_size)


def train_epoch(model, optimizer, sampler, x, y, train_nodes, batch_size, epoch=0, max_batches=None, on_batch=None):
    """One pass over `train_nodes` (int64, on the device) in a seeded random order. Returns the list of per-batch
    losses as a tensor on the device (no host synchronisation inside the loop besides the sampler's own).
    `on_batch(i, batch, loss)` is called after every step when given."""
    model.train()
    gen = torch.Generator(device=train_nodes.device).manual_seed(1234 + epoch)
    order = train_nodes[torch.randperm(train_nodes.shape[0], device=train_nodes.device, generator=gen)]
    total = num_batches(order.shape[0], batch_size)
    if max_batches is not None:
        total = min(total, max_batches)
    losses = torch.zeros(total, device=train_nodes.device)
    for b in range(total):
        seeds = order[b * batch_size:(b + 1) * batch_size]
        batch = sampler.batch(x, seeds, seed=epoch * 100003 + b, y=y)
        optimizer.zero_grad(set_to_none=True)
        out = model(batch)
        loss = F.nll_loss(out, batch.y)
        loss.backward()
        optimizer.step()
        losses[b] = loss.detach()
        if on_batch is not None:
            on_batch(b, batch, loss)
    return losses
