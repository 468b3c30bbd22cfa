"""Host-buffer entry points: the operators of this package applied to data that lives in
pinned HOST memory, with the host-to-device copies, the kernels and the device-to-host
copies of successive chunks overlapped on three CUDA streams.

A caller that keeps its arrays on the host pays PCIe for every byte in both directions;
issued on one stream (copy in, compute, copy out) the three phases add up.  Here a job is
cut into chunks (one dtype of a sweep, one sequence of a batch): chunk i's kernels wait for
chunk i's input copy only, and its output copy waits for its kernels only, so the upload of
chunk i+1 and the download of chunk i-1 run under chunk i's kernels, and uploads overlap
downloads (PCIe is full duplex).  A job then costs about max(upload, download) instead of
their sum.  The reference has no counterpart (its harnesses keep data on the device).

torch is used for streams, events and the copy calls; the kernels are this library's.
"""
from __future__ import annotations


class Chunk:
    """One unit of a pipelined job.
    h2d: list of (device_tensor, pinned_host_tensor) input copies;
    compute: callable that enqueues the chunk's kernels on the current stream;
    d2h: list of (pinned_host_tensor, device_tensor) result copies."""

    def __init__(self, h2d, compute, d2h):
        self.h2d, self.compute, self.d2h = list(h2d), compute, list(d2h)
        self.ev_in = self.ev_done = self.ev_out = None


class HostPipeline:
    """Runs a fixed list of chunks repeatedly.  Each run() enqueues everything and returns; the
    current stream is made to wait for the last copy, so a synchronize (or an event) on it
    covers the whole job.  Across runs, a chunk's upload waits for the kernels that read the
    same device buffers in the previous run, and its kernels for the previous download of
    their outputs."""

    def __init__(self, chunks, device=None):
        import torch
        self.torch = torch
        self.chunks = list(chunks)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=self.device) for _ in range(3))
        for c in self.chunks:
            for dst, src in c.h2d:
                if not src.is_pinned():
                    raise ValueError("input host tensors must be pinned")
            for dst, src in c.d2h:
                if not dst.is_pinned():
                    raise ValueError("output host tensors must be pinned")

    def bytes(self):
        n_in = sum(s.numel() * s.element_size() for c in self.chunks for _, s in c.h2d)
        n_out = sum(d.numel() * d.element_size() for c in self.chunks for d, _ in c.d2h)
        return n_in, n_out

    def run(self, compute: bool = True):
        """compute=False moves the same bytes and launches nothing: the copy floor of the job."""
        torch = self.torch
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        for c in self.chunks:
            with torch.cuda.stream(self.s_in):
                if c.ev_done is not None:
                    self.s_in.wait_event(c.ev_done)          # last run's kernels have read these buffers
                for dst, src in c.h2d:
                    dst.copy_(src, non_blocking=True)
                c.ev_in = torch.cuda.Event()
                c.ev_in.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(c.ev_in)
                if c.ev_out is not None:
                    self.s_run.wait_event(c.ev_out)          # last run's results have left the device
                if compute:
                    c.compute()
                c.ev_done = torch.cuda.Event()
                c.ev_done.record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(c.ev_done)
                for dst, src in c.d2h:
                    dst.copy_(src, non_blocking=True)
                c.ev_out = torch.cuda.Event()
                c.ev_out.record(self.s_out)
        for s in (self.s_in, self.s_run, self.s_out):
            end = torch.cuda.Event()
            end.record(s)
            cur.wait_event(end)


def segops_sweep_host(pkg, host_in: dict, jobs, device=None):
    """Pipeline for a sweep of segmented reduces / scans over pinned host arrays.
    host_in: {name: pinned 1-D tensor}; jobs: list of (name, "reduce" | "scan", op).
    One chunk per input array.  Returns (pipeline, {(name, fn, op): pinned result tensor})."""
    import torch
    device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    results, chunks = {}, []
    for name, h in host_in.items():
        mine = [(fn, op) for (n, fn, op) in jobs if n == name]
        if not mine:
            continue
        x = torch.empty(h.shape, dtype=h.dtype, device=device)
        outs = []
        for fn, op in mine:
            if fn == "reduce":
                odt = torch.float32 if h.dtype in (torch.float16, torch.bfloat16) else h.dtype
                o = torch.empty(h.numel() // 64, dtype=odt, device=device)
            else:
                o = torch.empty_like(x)
            ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()
            results[(name, fn, op)] = ho
            outs.append((fn, op, o, ho))

        def compute(x=x, outs=outs):
            for fn, op, o, _ in outs:
                (pkg.segreduce if fn == "reduce" else pkg.segscan)(x, op, out=o)

        chunks.append(Chunk([(x, h)], compute, [(ho, o) for _, _, o, ho in outs]))
    return HostPipeline(chunks, device), results


def prefill_host(pkg, Qh, Kh, Vh, causal: bool, Oh=None, device=None):
    """Pipeline for prefill attention over pinned host tensors Q [batch, nQH, seqQ, D] and
    K, V [batch, nKVH, seqK, D]: one chunk per sequence of the batch.  Returns (pipeline, Oh)."""
    import torch
    device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    if Oh is None:
        Oh = torch.empty(Qh.shape, dtype=Qh.dtype).pin_memory()
    chunks = []
    for b in range(Qh.shape[0]):
        q, k, v = (torch.empty(t[b:b + 1].shape, dtype=t.dtype, device=device) for t in (Qh, Kh, Vh))
        o = torch.empty_like(q)

        def compute(q=q, k=k, v=v, o=o):
            pkg.prefill(q, k, v, causal=causal, out=o)

        chunks.append(Chunk([(q, Qh[b:b + 1]), (k, Kh[b:b + 1]), (v, Vh[b:b + 1])], compute, [(Oh[b:b + 1], o)]))
    return HostPipeline(chunks, device), Oh
