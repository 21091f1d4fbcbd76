"""Layer forward for batches that live in host memory: the batch is cut into chunks and the
host-to-device copy of chunk i+1, the kernels of chunk i and the device-to-host copy of chunk i-1
run on three CUDA streams, so that the PCIe link is busy in both directions while the GPU works."""
import os

import torch

from . import ops


def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_host_node(index, sysfs="/sys/bus/pci/devices"):
    """(NUMA node, set of CPUs) next to GPU `index` as sysfs reports them for its PCI function, or (None, None)
    when that cannot be read (no sysfs entry, a virtual machine that hides the topology)."""
    try:
        pr = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
        base = os.path.join(sysfs, bdf)
        node = int(open(os.path.join(base, "numa_node")).read())
        cpus = _parse_cpulist(open(os.path.join(base, "local_cpulist")).read())
        return (node if node >= 0 else None), (cpus or None)
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None, None


def bind_to_gpu_node(index):
    """Restrict this process to the CPUs next to GPU `index`, so that the pinned host buffers it allocates afterwards
    (first touch) and the thread that feeds the copies sit on the GPU's NUMA node / PCIe root.  Call it before allocating
    pinned memory.  Returns what was done, for the record; binds nothing when the topology cannot be read or when the
    GPU's CPUs are all this process may use anyway."""
    node, cpus = gpu_host_node(index)
    allowed = os.sched_getaffinity(0)
    if not cpus:
        return {"numa_node": node, "bound": False, "why": "topology not readable", "cpus_allowed": len(allowed)}
    want = cpus & allowed
    if not want or want == allowed:
        return {"numa_node": node, "bound": False, "why": "the GPU's CPUs are all of this process's CPUs" if want else "no overlap",
                "cpus_allowed": len(allowed)}
    os.sched_setaffinity(0, want)
    return {"numa_node": node, "bound": True, "cpus": len(want), "cpus_allowed": len(allowed)}


class HostLayerPipeline:
    def __init__(self, B, H, W, C, K, layout="NHWC", math="tf32", relu=True, chunks=4, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.B, self.H, self.W, self.C, self.K = B, H, W, C, K
        self.layout, self.math, self.relu = layout, math, relu
        chunks = max(1, min(chunks, B))
        base, extra = divmod(B, chunks)
        self.bounds, lo = [], 0
        for i in range(chunks):
            hi = lo + base + (1 if i < extra else 0)
            self.bounds.append((lo, hi))
            lo = hi
        nH, nW = (H + 1) // 2, (W + 1) // 2
        in_shape = (lambda n: (n, H, W, C)) if layout == "NHWC" else (lambda n: (n, C, H, W))
        out_shape = (lambda n: (n, H, W, K)) if layout == "NHWC" else (lambda n: (n, K, H, W))
        with torch.cuda.device(self.device):
            self.xd = [torch.empty(in_shape(hi - lo), device=self.device) for lo, hi in self.bounds]
            self.yd = [torch.empty(out_shape(hi - lo), device=self.device) for lo, hi in self.bounds]
            biggest = max(hi - lo for lo, hi in self.bounds)
            self.vflat = [torch.empty(16 * biggest * nH * nW * C, device=self.device) for _ in range(2)]
            self.vshape = lambda n: (16, n, nH, nW, C)
            nws = ops.layer_fwd_prepared_workspace_bytes(biggest, H, W, C, K) if math == "tf32" else 0
            self.ws = torch.empty(nws, dtype=torch.uint8, device=self.device) if nws else None   # products of the wide path
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
            self.ev_in = [torch.cuda.Event() for _ in self.bounds]
            self.ev_run = [torch.cuda.Event() for _ in self.bounds]
            self.ev_out = [torch.cuda.Event() for _ in self.bounds]
        self._used = False
        self._prepared, self._prepared_for = None, None

    def _weights(self, Wt):
        if self.math != "tf32":
            return None
        key = (Wt.data_ptr(), Wt._version)
        if self._prepared_for != key:
            self._prepared = ops.prepare_weights(Wt)
            self._prepared_for = key
        return self._prepared

    def submit(self, x_host, Wt, y_host):
        """Enqueue one batch (pinned host x_host -> pinned host y_host) and return the CUDA event that marks its
        last device-to-host copy.  Calls may follow one another without waiting: the copies of the next batch
        overlap the kernels and the read-back of this one, so that in steady state the PCIe link is busy in both
        directions all the time.  Device buffers are reused across calls; the event dependencies below keep a
        chunk's buffers from being overwritten while the previous batch still uses them.  The caller must not
        reuse y_host (or change x_host) before the returned event has completed."""
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        self.s_run.wait_stream(cur)
        with torch.cuda.stream(self.s_run):
            prepared = self._weights(Wt)
        for i, (lo, hi) in enumerate(self.bounds):
            with torch.cuda.stream(self.s_in):
                if self._used:
                    self.s_in.wait_event(self.ev_run[i])      # the previous batch's kernels have read xd[i]
                self.xd[i].copy_(x_host[lo:hi], non_blocking=True)
                self.ev_in[i].record()
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.ev_in[i])
                if self._used:
                    self.s_run.wait_event(self.ev_out[i])     # the previous batch's yd[i] has been copied out
                shape = self.vshape(hi - lo)
                v = self.vflat[i % 2][:shape[0] * shape[1] * shape[2] * shape[3] * shape[4]].view(shape)
                if prepared is not None:
                    # the library picks the one-kernel path where it pays (v is then unused), else the two kernels
                    ops.layer_fwd_prepared(self.xd[i], prepared, self.K, relu=self.relu, layout=self.layout, out=self.yd[i],
                                           V_scratch=v, workspace=self.ws)
                else:
                    ops.imtrans_fwd(self.xd[i], relu=self.relu, layout=self.layout, out=v)
                    ops.conv_fwd(v, Wt, self.H, self.W, layout=self.layout, math=self.math, out=self.yd[i])
                self.ev_run[i].record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_run[i])
                y_host[lo:hi].copy_(self.yd[i], non_blocking=True)
                self.ev_out[i].record()
        self._used = True
        done = torch.cuda.Event()
        done.record(self.s_out)
        return done

    def __call__(self, x_host, Wt, y_host):
        """x_host, y_host: pinned host tensors of the full batch.  Returns y_host; it is complete once the
        caller's current stream has run past this call (e.g. after torch.cuda.current_stream().synchronize())."""
        done = self.submit(x_host, Wt, y_host)
        torch.cuda.current_stream(self.device).wait_event(done)
        return y_host
