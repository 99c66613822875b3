"""MoE layer passes whose tokens and results live in pinned HOST memory.

A caller that keeps activations on the host (an engine that runs the
attention part elsewhere, a test harness, a benchmark) pays a host->device copy
of the token rows and router logits and a device->host copy of the layer output
for every pass.  Issued on one stream those three steps run one after another;
`HostStagedMoe` gives each its own stream and a ring of device buffers, so pass
i+1's upload and pass i-1's download overlap pass i's kernels (PCIe is full
duplex, and the copies use the copy engines, not the SMs).  For the single-GPU
layer this class is a thin wrapper over the library's own runner
(gw_moe_host_runner_*, csrc/host_staged.cu); with a custom `run` callable (the
expert-parallel layers, which are driven from Python) the same staging is done
here with torch streams.

    runner = HostStagedMoe(workspace, table, expert_scales, max_rows, hidden)
    for batch in batches:
        runner.submit(batch.x, batch.scores, batch.y, rows)   # returns at once
    runner.synchronize()                                      # every batch.y is complete

The kernels of consecutive passes still run in order on the compute stream (a
workspace is one set of scratch buffers), and results are bit-identical to
`MoeWorkspace.run` on device buffers.

The runner's three streams are ordered among themselves only: weights, the
expert table and `expert_scales` must be complete on the device before the
first `submit` (synchronise the stream that prepared them), and the workspace
must not be used by other calls while passes are in flight.
"""
from __future__ import annotations

import ctypes

import torch

from .ops import ExpertTable, MoeWorkspace, _check, _library


class HostStagedMoe:
    def __init__(self, workspace: MoeWorkspace, table: ExpertTable, expert_scales: torch.Tensor, max_rows: int,
                 hidden: int, experts: int = 128, depth: int = 2, device=None, run=None, capture: bool = False):
        """`run(x, scores, y, rows, stream)`, when given, replaces `workspace.run` as the layer pass (the
        expert-parallel layers have their own entry point); it is called with the compute stream current
        and must issue all of its work on that stream.  With `capture`, the launches of `run` are recorded
        once per ring slot and row count in a CUDA graph and replayed afterwards (a pass of the
        expert-parallel layer is some thirty dependent launches: issued one by one from Python they, not
        the GPU, bound short passes); `run` must then read nothing back to the host and must have been
        called at least once before (its lazy initialisation cannot be recorded)."""
        if depth < 1:
            raise ValueError("depth must be at least 1")
        if not torch.cuda.is_available():
            raise RuntimeError("HostStagedMoe needs a CUDA device: there is no CPU execution path")
        self.workspace, self.table, self.expert_scales = workspace, table, expert_scales
        self.max_rows, self.hidden, self.experts, self.depth = max_rows, hidden, experts, depth
        self._run = run
        self._capture = bool(capture) and run is not None
        self._graphs = {}
        device = device if device is not None else expert_scales.device
        self.device = device
        self._native = None
        self._submitted = 0
        if run is None:
            if hidden != 2816 or experts != 128:
                raise ValueError("the library's runner is built for hidden 2816 and 128 experts")
            self._lib = _library()
            self._native = ctypes.c_void_p()
            _check(self._lib.gw_moe_host_runner_create(workspace._ws, table.handle, expert_scales.data_ptr(), max_rows,
                                                       depth, ctypes.byref(self._native)))
            streams = [ctypes.c_void_p() for _ in range(3)]
            _check(self._lib.gw_moe_host_runner_streams(self._native, *(ctypes.byref(s) for s in streams)))
            self.upload, self.compute, self.download = (torch.cuda.ExternalStream(s.value, device=device)
                                                        for s in streams)
            return
        self.upload, self.compute, self.download = (torch.cuda.Stream(device=device) for _ in range(3))
        self._x = [torch.empty((max_rows, hidden), dtype=torch.bfloat16, device=device) for _ in range(depth)]
        self._scores = [torch.empty((max_rows, experts), dtype=torch.bfloat16, device=device) for _ in range(depth)]
        self._y = [torch.empty((max_rows, hidden), dtype=torch.bfloat16, device=device) for _ in range(depth)]
        # per slot: the pass that last used it has finished computing / downloading
        self._computed = [None] * depth
        self._downloaded = [None] * depth
        self._h2d = 0
        self._d2h = 0

    @property
    def h2d_bytes(self) -> int:
        return int(self._lib.gw_moe_host_runner_h2d_bytes(self._native)) if self._native else self._h2d

    @property
    def d2h_bytes(self) -> int:
        return int(self._lib.gw_moe_host_runner_d2h_bytes(self._native)) if self._native else self._d2h

    def submit(self, host_x: torch.Tensor, host_scores: torch.Tensor, host_y: torch.Tensor, rows: int) -> int:
        """Queue one layer pass: host_x [rows, hidden] and host_scores [rows, experts] (BF16, pinned) are
        uploaded, the layer runs, the output lands in host_y [rows, hidden] (BF16, pinned).  Returns the
        pass's sequence number without waiting; `synchronize()` (or `wait_for`) makes host_y readable."""
        if rows < 0 or rows > self.max_rows:
            raise ValueError(f"rows = {rows} outside [0, {self.max_rows}]")
        for name, t, width in (("host_x", host_x, self.hidden), ("host_scores", host_scores, self.experts),
                               ("host_y", host_y, self.hidden)):
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError(f"{name} must be a pinned host tensor")
            if t.dtype != torch.bfloat16 or t.dim() != 2 or t.shape[1] != width or t.shape[0] < rows \
                    or not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous BF16 [>= rows, {width}]")
        if self._native:
            ticket = ctypes.c_uint64()
            _check(self._lib.gw_moe_host_runner_submit(self._native, host_x.data_ptr(), host_scores.data_ptr(),
                                                       host_y.data_ptr(), rows, ctypes.byref(ticket)))
            self._submitted = ticket.value + 1
            return int(ticket.value)
        ticket = self._submitted
        slot = ticket % self.depth
        x, scores, y = self._x[slot], self._scores[slot], self._y[slot]
        if rows > 0 or self._run is not None:     # a rank without rows still serves its experts in a custom pass
            with torch.cuda.stream(self.upload):
                if self._computed[slot] is not None:        # the slot's previous pass no longer reads its inputs
                    self.upload.wait_event(self._computed[slot])
                x[:rows].copy_(host_x[:rows], non_blocking=True)
                scores[:rows].copy_(host_scores[:rows], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self.upload)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(uploaded)
                if self._downloaded[slot] is not None:      # the slot's previous output has left the device
                    self.compute.wait_event(self._downloaded[slot])
                if self._capture:
                    graph = self._graphs.get((slot, rows))
                    if graph is None:
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph, stream=self.compute, capture_error_mode="thread_local"):
                            self._run(x, scores, y, rows, self.compute)
                        self._graphs[(slot, rows)] = graph
                    graph.replay()
                elif self._run is not None:
                    self._run(x, scores, y, rows, self.compute)
                else:
                    self.workspace.run(x, scores, self.expert_scales, self.table, y, rows, stream=self.compute)
                computed = torch.cuda.Event()
                computed.record(self.compute)
            with torch.cuda.stream(self.download):
                self.download.wait_event(computed)
                host_y[:rows].copy_(y[:rows], non_blocking=True)
                downloaded = torch.cuda.Event()
                downloaded.record(self.download)
            self._computed[slot], self._downloaded[slot] = computed, downloaded
            self._h2d += rows * (self.hidden + self.experts) * 2
            self._d2h += rows * self.hidden * 2
        self._submitted += 1
        return ticket

    def wait_for(self, ticket: int) -> None:
        """Block the host until pass `ticket`'s output is in its host buffer."""
        if ticket < 0 or ticket >= self._submitted:
            raise ValueError("no such pass")
        if self._native:
            _check(self._lib.gw_moe_host_runner_wait(self._native, ticket))
            return
        # the download stream runs in order: the newest download queued on the pass's slot is not
        # earlier than the pass's own
        event = self._downloaded[ticket % self.depth]
        if event is not None:
            event.synchronize()

    def synchronize(self) -> None:
        if self._native:
            _check(self._lib.gw_moe_host_runner_synchronize(self._native))
            return
        for stream in (self.upload, self.compute, self.download):
            stream.synchronize()

    def __del__(self):
        if getattr(self, "_native", None):
            self._lib.gw_moe_host_runner_destroy(self._native)
            self._native = None
