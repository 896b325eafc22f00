"""HostStream: chunked host<->device pipeline gives the same result as copy-all,
compute, copy-all, also when steps follow each other."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_stream_matches_plain_copies():
    from nntile_b200.parallel import HostStream
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(5)
    units, inner = 6, 1 << 18
    host_a = torch.randn((units, inner), generator=g).pin_memory()
    host_b = torch.randn((units, inner), generator=g).pin_memory()
    host_o = torch.empty((units, inner)).pin_memory()
    dev_a, dev_b = (torch.empty((units, inner), device=dev) for _ in range(2))
    dev_o = torch.zeros((units, inner), device=dev)

    def body(lo, hi):
        # several dependent kernels per chunk, accumulating like the "+=" outputs do
        t = dev_a[lo:hi]*2.0
        t = t + dev_b[lo:hi]
        dev_o[lo:hi] += t

    pipe = HostStream(dev, units, chunks=4)
    want = torch.zeros((units, inner))
    for step in range(3):
        host_a.mul_(1.5)            # the host changes its inputs between steps
        want += host_a*2.0 + host_b
        pipe.step((host_a, host_b), (dev_a, dev_b), body, (dev_o,), (host_o,))
        torch.cuda.synchronize()
        assert torch.allclose(host_o, want, rtol=1e-5, atol=1e-5), f"step {step}"


def test_host_stream_pipelines_steps_without_a_sync_in_between():
    """Steps enqueued back to back (the copy-in of step k+1 overlaps the copy-out of
    step k) give the same result as synchronised ones; join() ends the pipeline."""
    from nntile_b200.parallel import HostStream
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(6)
    units, inner, steps = 8, 1 << 20, 5
    host_a = torch.randn((units, inner), generator=g).pin_memory()
    host_o = torch.empty((units, inner)).pin_memory()
    dev_a = torch.empty((units, inner), device=dev)
    dev_o = torch.zeros((units, inner), device=dev)

    def body(lo, hi):
        dev_o[lo:hi] += dev_a[lo:hi]*0.5
        dev_a[lo:hi].zero_()                    # a stale input would show in the next step

    pipe = HostStream(dev, units, chunks=4)
    for _ in range(steps):
        pipe.step((host_a,), (dev_a,), body, (dev_o,), (host_o,))
    pipe.join()
    torch.cuda.synchronize()
    assert torch.allclose(host_o, host_a*(0.5*steps), rtol=1e-5, atol=1e-5)
    # after join() a new pipeline starts cleanly
    pipe.step((host_a,), (dev_a,), body, (dev_o,), (host_o,))
    pipe.join()
    torch.cuda.synchronize()
    assert torch.allclose(host_o, host_a*(0.5*(steps + 1)), rtol=1e-5, atol=1e-5)
