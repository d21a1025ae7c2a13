"""Host-buffer front end: points in pinned host memory in, harmonics in pinned host memory out.

This is the call a user with NumPy-side data makes (the reference's NumPy path,
``python/src/sphericart/spherical_harmonics.py:101-138``, takes host arrays and returns host
arrays). The points are cut into chunks; each chunk is copied to the device, evaluated by the
CUDA library and copied back on one of several streams, so the device-to-host copy of one chunk
overlaps the host-to-device copy and the kernel of the next. The outputs are ~100x larger than
the inputs, so this path is bound by the PCIe device-to-host bandwidth, not by the kernel.
"""

import torch


class HostPipeline:
    def __init__(self, calculator, level, dtype, device, chunk_points=1 << 18, n_streams=3):
        self.calc = calculator
        self.level = int(level)
        self.dtype = dtype
        self.device = torch.device(device)
        self.chunk = int(chunk_points)
        ny = (calculator.l_max + 1) ** 2
        self.ny = ny
        self.streams = [torch.cuda.Stream(device=self.device) for _ in range(n_streams)]
        shapes = [(self.chunk, ny), (self.chunk, 3, ny), (self.chunk, 3, 3, ny)][: self.level + 1]
        self.bufs = []
        for _ in self.streams:
            xyz = torch.empty((self.chunk, 3), dtype=dtype, device=self.device)
            outs = [torch.empty(s, dtype=dtype, device=self.device) for s in shapes]
            self.bufs.append((xyz, outs))
        self.launches = 0

    def bytes_per_point(self):
        size = torch.empty((), dtype=self.dtype).element_size()
        return 3 * size, self.ny * (1, 4, 13)[self.level] * size

    def run(self, xyz_host, outs_host):
        """xyz_host: pinned (n, 3); outs_host: pinned outputs [(n, ny), (n, 3, ny), ...]. Blocks until done."""
        n = xyz_host.shape[0]
        caller = torch.cuda.current_stream(self.device)
        for s in self.streams:
            s.wait_stream(caller)
        for ci, lo in enumerate(range(0, n, self.chunk)):
            hi = min(n, lo + self.chunk)
            m = hi - lo
            stream = self.streams[ci % len(self.streams)]
            d_xyz, d_outs = self.bufs[ci % len(self.streams)]
            with torch.cuda.stream(stream):
                d_xyz[:m].copy_(xyz_host[lo:hi], non_blocking=True)
                self.calc.compute_raw(self.dtype, self.level, d_xyz.data_ptr(), m, d_outs[0].data_ptr(),
                                      d_outs[1].data_ptr() if self.level >= 1 else None,
                                      d_outs[2].data_ptr() if self.level >= 2 else None, stream.cuda_stream)
                self.launches += 1
                for d, h in zip(d_outs, outs_host):
                    h[lo:hi].copy_(d[:m], non_blocking=True)
        for s in self.streams:
            caller.wait_stream(s)
        caller.synchronize()
