import torch


def compare(output1, output2, atol=1e-2, rtol=1e-2):
    """Agreement report of the reference (cxgnncomp/codegen/util.py:5-15): prints and returns the verdict."""
    assert output1.shape == output2.shape, f"{output1.shape} != {output2.shape}"
    ok = bool(torch.allclose(output1, output2, atol=atol, rtol=rtol))
    print("CORRECT: match" if ok else "ERROR: differ")
    return ok


def prof(name, tag, func, warmup=3, rep=10):
    """Median milliseconds of func() measured with CUDA events (the reference uses triton.testing.do_bench,
    cxgnncomp/codegen/util.py:18-29, and reports its median)."""
    for _ in range(warmup):
        func()
    times = []
    for _ in range(rep):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        func()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    med = times[len(times) // 2]
    print(f"{name} {tag} {med:.4f} ms")
    return med, times[0], times[-1]
