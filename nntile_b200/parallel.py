"""Sharding of the path over one process per GPU.

Every (batch, kv head) slice of the SDPA tensors is an independent attention
problem (src/tensor/flash_sdpa_fwd_cudnn.cc:221-233: the outer loop runs over
output tiles, only the inner K/V-sequence loop carries a dependency), which is
how the reference spreads tile tasks over StarPU CUDA workers.  Here the units
are dealt out in contiguous blocks, one block per rank, and no collective sits
on the data path; ``regather`` is the optional all-gather for a caller that
wants the whole output on every rank.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block [lo, hi) of `n_units` for `rank`; sizes differ by at most 1."""
    if world <= 0 or not (0 <= rank < world) or n_units < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n_units, world)
    lo = rank*base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_units(tensor: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Slice a (kv_heads, group, batch, ...) buffer by (kv head, batch) units.

    Units are numbered kv_head*batch + b; a rank's block must not split a kv
    head unevenly across the batch axis unless it covers whole batches, so the
    split is done on the kv-head axis when it divides and on the batch axis
    otherwise."""
    H, G, B = tensor.shape[:3]
    if H % world == 0:
        lo, hi = shard_range(H, rank, world)
        return tensor[lo:hi]
    if B % world == 0:
        lo, hi = shard_range(B, rank, world)
        return tensor[:, :, lo:hi]
    raise ValueError(f"neither kv_heads={H} nor batch={B} divides over {world} ranks")


def regather(local: torch.Tensor, axis: int = 0, group=None) -> torch.Tensor:
    """All-gather equally sized shards along `axis` (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=axis)


def max_over_ranks(value: float, device, group=None) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def chunk_ranges(n_units: int, chunks: int) -> list[tuple[int, int]]:
    """[lo, hi) blocks of the leading (kv head) index for `chunks` pipeline stages."""
    chunks = max(1, min(int(chunks), int(n_units)))
    return [shard_range(n_units, c, chunks) for c in range(chunks)]


class HostStream:
    """Runs a per-unit body on tensors that live in pinned host memory, with the
    copies overlapped with the kernels - inside a step and from one step to the next.

    The reference leaves this to StarPU: its codelets are STARPU_CUDA_ASYNC
    (src/starpu/codelet.cc:80), so the runtime moves the next task's handles to the
    GPU and the previous task's results back while a task computes.  Here the
    leading index of the buffers (independent units) is cut into chunks and three
    streams are chained by events, chunk by chunk: host-to-device copy of a chunk,
    its kernels, device-to-host copy of its results.  Nothing waits for a whole
    step: the copy-in of chunk c of step k+1 only waits for the kernels of chunk c
    of step k (which read the same device buffers), and those kernels only wait for
    the copy-out of chunk c of step k.  PCIe is full duplex, so a stream of steps
    costs about max(copy in, copy out) per step instead of copy in + kernels +
    copy out.  `join()` makes the current stream wait for the last results.

    `body(lo, hi)` enqueues the kernels for units [lo, hi) on the current stream;
    all tensors are indexed by unit along axis 0."""

    def __init__(self, device, n_units: int, chunks: int = 8):
        self.device = device
        self.ranges = chunk_ranges(n_units, chunks)
        self.s_in = torch.cuda.Stream(device=device)
        self.s_out = torch.cuda.Stream(device=device)
        self.ev_in = [torch.cuda.Event() for _ in self.ranges]
        self.ev_done = [torch.cuda.Event() for _ in self.ranges]
        self.ev_out = [torch.cuda.Event() for _ in self.ranges]
        self.started = False

    def step(self, host_in, dev_in, body, dev_out, host_out):
        cur = torch.cuda.current_stream(self.device)
        if not self.started:
            # whatever filled or still reads the device buffers comes first
            self.s_in.wait_stream(cur)
            self.s_out.wait_stream(cur)
        for c, (lo, hi) in enumerate(self.ranges):
            if self.started:
                self.s_in.wait_event(self.ev_done[c])     # last step's kernels read dev_in[c]
            with torch.cuda.stream(self.s_in):
                for h, d in zip(host_in, dev_in):
                    d[lo:hi].copy_(h[lo:hi], non_blocking=True)
                self.ev_in[c].record(self.s_in)
        for c, (lo, hi) in enumerate(self.ranges):
            cur.wait_event(self.ev_in[c])
            if self.started:
                cur.wait_event(self.ev_out[c])            # last step's results have left dev_out[c]
            body(lo, hi)
            self.ev_done[c].record(cur)
            self.s_out.wait_event(self.ev_done[c])
            with torch.cuda.stream(self.s_out):
                for h, d in zip(host_out, dev_out):
                    h[lo:hi].copy_(d[lo:hi], non_blocking=True)
                self.ev_out[c].record(self.s_out)
        self.started = True

    def join(self):
        """The current stream waits until every result enqueued so far is on the host
        (and every copy-in is done); the next step() starts a fresh pipeline."""
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)
        self.started = False
