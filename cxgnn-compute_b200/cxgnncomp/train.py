"""Mini-batch epoch loop over sampled CSR_Layer batches: sample -> gather features -> forward -> NLL loss on the
seeds -> backward -> optimizer step (the reference's Trainer.cxg_train_epoch, cxgnncomp/trainer.py:140-175, with
the sampler of this package in place of its external loader)."""
import math
import queue
import threading

import torch
import torch.nn.functional as F


def num_batches(num_train, batch_size):
    return math.ceil(num_train / batch_size)


def train_epoch(model, optimizer, sampler, x, y, train_nodes, batch_size, epoch=0, max_batches=None, on_batch=None,
                prefetch=True, depth=2):
    """One pass over `train_nodes` (int64, on the device) in a seeded random order. Returns the list of per-batch
    losses as a tensor on the device. `on_batch(i, batch, loss)` is called after every step when given.

    prefetch (CUDA only): True = a producer thread samples the batches ahead (at most `depth` waiting) on a side
    stream while this thread issues the training steps, so neither the sampler's host synchronisations (it reads
    two counts per hop) nor its host work sit between two training steps; "stream" = sample batch b + 1 on a side
    stream from this thread before issuing step b (device work overlaps, host work does not); False = everything
    in order on the current stream. Same batches, same losses in all three."""
    model.train()
    gen = torch.Generator(device=train_nodes.device).manual_seed(1234 + epoch)
    order = train_nodes[torch.randperm(train_nodes.shape[0], device=train_nodes.device, generator=gen)]
    total = num_batches(order.shape[0], batch_size)
    if max_batches is not None:
        total = min(total, max_batches)
    losses = torch.zeros(total, device=train_nodes.device)
    if not (train_nodes.is_cuda and total > 0):
        prefetch = False
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
    producer, stop, q = None, None, None
    if prefetch is True:
        q, stop = queue.Queue(maxsize=max(1, int(depth))), threading.Event()
        device = train_nodes.device

        def offer(item):
            """Puts `item` unless the consumer has gone; never blocks for good."""
            while not stop.is_set():
                try:
                    q.put(item, timeout=0.1)
                    return True
                except queue.Full:
                    pass
            return False

        def run():
            try:
                with torch.cuda.device(device):
                    for b in range(total):
                        if not offer(produce(b)):
                            return
            except BaseException as e:  # handed to the consumer, which re-raises it
                offer(e)

        producer = threading.Thread(target=run, name="cxg-batch-producer", daemon=True)
        producer.start()
    try:
        nxt = produce(0) if (total > 0 and producer is None) else None
        for b in range(total):
            if producer is not None:
                item = q.get()
                if isinstance(item, BaseException):
                    raise item
                batch, ready = item
            else:
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
    finally:
        if producer is not None:
            stop.set()
            producer.join()
    if prefetch:
        side.wait_stream(main)
    return losses
