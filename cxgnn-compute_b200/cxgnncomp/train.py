"""Mini-batch epoch loop over sampled CSR_Layer batches: sample -> gather features -> forward -> NLL loss on the
seeds -> backward -> optimizer step (the reference's Trainer.cxg_train_epoch, cxgnncomp/trainer.py:140-175, with
the sampler of this package in place of its external loader)."""
import math

import torch
import torch.nn.functional as F


def num_batches(num_train, batch_size):
    return math.ceil(num_train / batch_size)


def train_epoch(model, optimizer, sampler, x, y, train_nodes, batch_size, epoch=0, max_batches=None, on_batch=None,
                prefetch=True):
    """One pass over `train_nodes` (int64, on the device) in a seeded random order. Returns the list of per-batch
    losses as a tensor on the device. `on_batch(i, batch, loss)` is called after every step when given.

    prefetch=True (CUDA only) samples batch b + 1 on a side stream while the model trains on batch b: the sampler's
    host synchronisations (it reads two counts per hop) then wait for the short sampling work only, not for the
    training step queued before them, and sampling overlaps training on the device. Same batches, same losses."""
    model.train()
    gen = torch.Generator(device=train_nodes.device).manual_seed(1234 + epoch)
    order = train_nodes[torch.randperm(train_nodes.shape[0], device=train_nodes.device, generator=gen)]
    total = num_batches(order.shape[0], batch_size)
    if max_batches is not None:
        total = min(total, max_batches)
    losses = torch.zeros(total, device=train_nodes.device)
    prefetch = prefetch and train_nodes.is_cuda and total > 0
    main = torch.cuda.current_stream() if prefetch else None
    side = torch.cuda.Stream() if prefetch else None

    def produce(b):
        seeds = order[b * batch_size:(b + 1) * batch_size]
        if not prefetch:
            return sampler.batch(x, seeds, seed=epoch * 100003 + b, y=y), None
        with torch.cuda.stream(side):
            batch = sampler.batch(x, seeds, seed=epoch * 100003 + b, y=y)
            ready = torch.cuda.Event()
            ready.record(side)
        return batch, ready

    if prefetch:
        side.wait_stream(main)  # `order` and the model's inputs were produced on the main stream
    nxt = produce(0) if total > 0 else None
    for b in range(total):
        batch, ready = nxt
        if b + 1 < total:
            nxt = produce(b + 1)
        if ready is not None:
            main.wait_event(ready)
            for t in (batch.x, batch.ptr, batch.idx, batch.y, batch.target):
                if isinstance(t, torch.Tensor):
                    t.record_stream(main)  # allocated on the side stream, used on the main one
        optimizer.zero_grad(set_to_none=True)
        out = model(batch)
        loss = F.nll_loss(out, batch.y)
        loss.backward()
        optimizer.step()
        losses[b] = loss.detach()
        if on_batch is not None:
            on_batch(b, batch, loss)
    if prefetch:
        side.wait_stream(main)
    return losses
