"""Expert-parallel execution of the 128-expert / top-8 MoE layer over the GPUs
of one node (one process per GPU, torch.distributed for the plumbing).

The reference runs this layer on a single GPU (sm120::MoeWorkspace,
models/gemma4/26b_a4b/sm120/moe.cu:462-545); sharding it by expert is new here.
Experts are placed contiguously (expert e lives on rank e // (128 / R)); every
rank owns T / R tokens and

  1. routes its own tokens (bit-exact with the single-GPU routing, no traffic),
  2. exchanges the per-expert row counts (R x 128/R integers each way),
  3. sends its rows, sorted by expert and therefore by destination rank, with
     one all-to-all-v (dispatch),
  4. runs the grouped gate/up GEMM -> GeGLU -> grouped down GEMM over the rows
     it received, read through an index that regroups them expert-major,
  5. returns the results with the mirrored all-to-all-v (combine traffic) and
  6. folds the eight weighted rows of each token in ascending expert order
     (moe.cu:446-456), exactly as the single-GPU layer does.

Every per-row operation is the same kernel as on one GPU, so the result is
independent of the number of ranks.

The class is written against a small backend interface so that the exchange
logic (counts, splits, regrouping permutation) can be exercised on CPU ranks
with the gloo backend; the product backend (`DeviceBackend`) calls the CUDA
library and nothing else.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

EXPERTS, TOPK, HIDDEN, INTER = 128, 8, 2816, 704


def owner_of(expert: int, world: int) -> int:
    """Contiguous placement: 128 / world experts per rank."""
    return expert // (EXPERTS // world)


def local_expert_range(rank: int, world: int) -> range:
    per_rank = EXPERTS // world
    return range(rank * per_rank, (rank + 1) * per_rank)


@dataclass
class ExchangeLayout:
    """How the rows a rank received (ordered by source rank, then expert) map
    onto the expert-major order the grouped GEMMs want."""
    total: int                    # rows received
    dest_of_source: torch.Tensor  # int32 [total]: expert-major position of received row j
    source_of_dest: torch.Tensor  # int32 [total]: received row that expert-major row i reads
    local_offsets: torch.Tensor   # int32 [experts_per_rank + 1]: expert-major group boundaries


def exchange_layout(recv_counts: torch.Tensor, total: int) -> ExchangeLayout:
    """recv_counts[s, e] = rows source rank s sends for this rank's local expert e.

    Received rows arrive as [s][e][k]; the expert-major order is [e][s][k] (a
    stable regrouping, so rows of one expert keep source-rank-then-token
    order).  Pure tensor arithmetic on the counts' device; `total` is their sum
    (known on the host from the split sizes)."""
    counts = recv_counts.to(torch.int64)
    sources, experts = counts.shape
    per_expert = counts.sum(0)
    local_offsets = torch.zeros(experts + 1, dtype=torch.int64, device=counts.device)
    local_offsets[1:] = per_expert.cumsum(0)
    flat = counts.reshape(-1)                                     # [s * experts + e]
    source_start = flat.cumsum(0) - flat                          # start of segment (s, e) in arrival order
    within_expert = counts.cumsum(0) - counts                     # rows of expert e from sources < s
    dest_start = (local_offsets[:-1].unsqueeze(0) + within_expert).reshape(-1)
    if total == 0:
        empty = torch.empty(0, dtype=torch.int32, device=counts.device)
        return ExchangeLayout(0, empty, empty.clone(), local_offsets.to(torch.int32))
    segment = torch.repeat_interleave(torch.arange(sources * experts, device=counts.device), flat, output_size=total)
    arrival = torch.arange(total, device=counts.device)
    dest_of_source = dest_start[segment] + (arrival - source_start[segment])
    source_of_dest = torch.empty_like(dest_of_source)
    source_of_dest[dest_of_source] = arrival
    return ExchangeLayout(total, dest_of_source.to(torch.int32), source_of_dest.to(torch.int32),
                          local_offsets.to(torch.int32))


class DeviceBackend:
    """The CUDA library as the per-rank engine.  `experts` has 128 entries,
    (gate, up, down) NVFP4 weights for the experts this rank owns and None for
    the others."""

    def __init__(self, experts, local_tokens: int, receive_capacity_rows: int):
        import gewell_b200 as gw
        self.gw = gw
        self.table = gw.ExpertTable(experts)
        self.route_ws = gw.MoeWorkspace(local_tokens)
        self.expert_ws = gw.MoeWorkspace((receive_capacity_rows + 7) // 8)
        self.device = self.route_ws.device

    def empty_rows(self, rows: int) -> torch.Tensor:
        return torch.empty((rows, HIDDEN), dtype=torch.bfloat16, device=self.device)

    def route(self, scores, expert_scales, rows: int):
        self.route_ws.dispatch(scores, expert_scales, rows)
        return self.route_ws.routing_state(rows)

    def gather(self, x, index, divisor: int, rows: int, out):
        self.gw.ops._check(self.gw.lib.gw_gather_rows_bf16(x.data_ptr(), index.data_ptr(), divisor, rows, HIDDEN,
                                                           out.data_ptr(), torch.cuda.current_stream().cuda_stream))
        return out

    def experts(self, rows_in, row_index, local_offsets, first_expert: int, expert_count: int, total: int, out):
        self.expert_ws.run_sorted(rows_in, local_offsets, first_expert, expert_count, total, self.table, out,
                                  row_index=row_index)
        return out

    def combine(self, down_rows, inverse, weights, rows: int, out):
        self.gw.ops._check(self.gw.lib.gw_moe_combine(down_rows.data_ptr(), inverse.data_ptr(), weights.data_ptr(),
                                                      rows, HIDDEN, out.data_ptr(),
                                                      torch.cuda.current_stream().cuda_stream))
        return out


class Placement:
    """Which rank owns which expert.  Every rank owns 128 / R experts; inside a
    rank they are kept in ascending id order.  `physical[e]` is the position of
    expert e in the (rank, id) order: a rank's expert table is indexed by
    physical position, and rows travel grouped by physical position."""

    def __init__(self, owner: list[int], world: int):
        if len(owner) != EXPERTS or EXPERTS % world:
            raise ValueError("placement needs one owner per expert and a rank count that divides 128")
        per_rank = EXPERTS // world
        if any(sum(1 for o in owner if o == r) != per_rank for r in range(world)):
            raise ValueError("every rank must own exactly 128 / R experts")
        self.world, self.per_rank, self.owner = world, per_rank, list(owner)
        self.order = sorted(range(EXPERTS), key=lambda e: (owner[e], e))       # physical position -> expert id
        self.physical = [0] * EXPERTS
        for position, e in enumerate(self.order):
            self.physical[e] = position

    @staticmethod
    def contiguous(world: int) -> "Placement":
        return Placement([owner_of(e, world) for e in range(EXPERTS)], world)

    @staticmethod
    def interleaved(world: int) -> "Placement":
        """expert e on rank e % R: spreads a popularity that falls with the id."""
        return Placement([e % world for e in range(EXPERTS)], world)

    @staticmethod
    def balanced(world: int, load: list[float]) -> "Placement":
        """Load-aware placement from a measured per-expert row count (for
        instance the routing histogram of earlier batches): experts in order of
        falling load each go to the rank with the least load so far that still
        has a free slot (longest-processing-time rule)."""
        if len(load) != EXPERTS:
            raise ValueError("one load figure per expert")
        per_rank = EXPERTS // world
        totals, slots, owner = [0.0] * world, [0] * world, [0] * EXPERTS
        for e in sorted(range(EXPERTS), key=lambda e: (-load[e], e)):
            rank = min((r for r in range(world) if slots[r] < per_rank), key=lambda r: (totals[r], r))
            owner[e] = rank
            totals[rank] += load[e]
            slots[rank] += 1
        return Placement(owner, world)

    def local_experts(self, rank: int) -> list[int]:
        return self.order[rank * self.per_rank:(rank + 1) * self.per_rank]


class ExpertParallelMoe:
    """One rank's share of the expert-parallel layer.  `backend` supplies
    route / gather / experts / combine / empty_rows (see DeviceBackend); its
    expert table is indexed by physical position (see Placement)."""

    STAGES = ("route", "counts", "gather", "dispatch_all_to_all", "experts", "regroup", "combine_all_to_all",
              "combine")

    def __init__(self, backend, rank: int, world: int, local_tokens: int, receive_capacity_rows: int, group=None,
                 placement: Placement | None = None):
        self.placement = placement or Placement.contiguous(world)
        if self.placement.world != world:
            raise ValueError("placement was built for another number of ranks")
        self.backend, self.rank, self.world, self.group = backend, rank, world, group
        self.local_tokens, self.capacity = local_tokens, receive_capacity_rows
        self.per_rank = EXPERTS // world
        n = TOPK * local_tokens
        self.send_rows = backend.empty_rows(n)
        self.returned_rows = backend.empty_rows(n)
        self.received = backend.empty_rows(receive_capacity_rows)
        self.expert_out = backend.empty_rows(receive_capacity_rows)
        self.expert_out_arrival = backend.empty_rows(receive_capacity_rows)
        device = self.send_rows.device
        self.order = torch.tensor(self.placement.order, dtype=torch.int64, device=device)
        self.physical = torch.tensor(self.placement.physical, dtype=torch.int64, device=device)
        self.identity = self.placement.order == list(range(EXPERTS))
        self.last_layout: ExchangeLayout | None = None
        self.last_splits = None
        self.timer = None      # optional callable(stage_name), called after each stage is enqueued

    def _mark(self, name: str):
        if self.timer is not None:
            self.timer(name)

    def run(self, x, scores, expert_scales, rows: int, out=None):
        """x [rows, 2816] BF16, scores [rows, 128] BF16 router logits,
        expert_scales [128] BF16; returns the layer output [rows, 2816] BF16 for
        this rank's tokens."""
        if rows > self.local_tokens:
            raise ValueError("more tokens than this rank was sized for")
        b, world = self.backend, self.world
        n = TOPK * rows
        offsets, sorted_assignments, inverse, weights = b.route(scores, expert_scales, rows)
        self._mark("route")
        # rows per (destination rank, its local expert), exchanged so that every rank
        # learns what it will receive; the split sizes are needed on the host
        counts = (offsets[1:] - offsets[:-1]).to(torch.int64)
        send_counts = counts[self.order].reshape(world, self.per_rank).to(torch.int32).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sizes = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
        send_splits, recv_splits = sizes[0].tolist(), sizes[1].tolist()
        total = int(sum(recv_splits))
        if total > self.capacity:
            raise RuntimeError(f"rank {self.rank} would receive {total} rows but was sized for {self.capacity}")
        layout = exchange_layout(recv_counts, total)
        self.last_layout, self.last_splits = layout, (send_splits, recv_splits)
        if self.identity:
            send_source, home = sorted_assignments, inverse
        else:
            # the routing sorted the rows by expert id; they travel sorted by physical
            # position: shift every expert's segment to its place in the send order
            flat = send_counts.reshape(-1).to(torch.int64)
            send_start = flat.cumsum(0) - flat                                  # by physical position
            shift = send_start[self.physical] - offsets[:-1].to(torch.int64)     # by expert id
            keys = torch.repeat_interleave(torch.arange(EXPERTS, device=counts.device), counts, output_size=n)
            send_position = torch.arange(n, device=counts.device) + shift[keys]
            send_source = torch.empty(n, dtype=torch.int32, device=counts.device)
            send_source[send_position] = sorted_assignments[:n]
            home = send_position[inverse[:n].to(torch.int64)].to(torch.int32)
        self._mark("counts")
        # dispatch: rows in send order are contiguous per destination rank
        b.gather(x, send_source, TOPK, n, self.send_rows)
        self._mark("gather")
        dist.all_to_all_single(self.received[:total], self.send_rows[:n], recv_splits, send_splits, group=self.group)
        self._mark("dispatch_all_to_all")
        first = self.rank * self.per_rank
        b.experts(self.received, layout.source_of_dest, layout.local_offsets, first, self.per_rank, total,
                  self.expert_out)
        self._mark("experts")
        # back to arrival order, then home
        b.gather(self.expert_out, layout.dest_of_source, 1, total, self.expert_out_arrival)
        self._mark("regroup")
        dist.all_to_all_single(self.returned_rows[:n], self.expert_out_arrival[:total], send_splits, recv_splits,
                               group=self.group)
        self._mark("combine_all_to_all")
        if out is None:
            out = b.empty_rows(rows)
        b.combine(self.returned_rows, home, weights, rows, out)
        self._mark("combine")
        return out


class SharedBuffer:
    """Device memory that every rank of the node can address: each rank
    allocates its own buffer (gw_ipc_alloc), the 64-byte handles are exchanged
    through the process group, and every rank maps the others' buffers
    (gw_ipc_open).  `pointers[r]` is rank r's buffer as seen from this process."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        import ctypes
        import gewell_b200 as gw
        self._gw, self.rank, self.world, self.nbytes = gw, rank, world, nbytes
        pointer, handle = ctypes.c_void_p(), (ctypes.c_uint8 * 64)()
        gw.ops._check(gw.lib.gw_ipc_alloc(nbytes, ctypes.byref(pointer), handle))
        self.local = pointer.value
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.pointers = []
        for r in range(world):
            if r == rank:
                self.pointers.append(self.local)
                continue
            peer = ctypes.c_void_p()
            raw = (ctypes.c_uint8 * 64).from_buffer_copy(handles[r])
            gw.ops._check(gw.lib.gw_ipc_open(raw, ctypes.byref(peer)))
            self.pointers.append(peer.value)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.pointer_table = torch.tensor(self.pointers, dtype=torch.int64, device=self.device)

    def close(self, group=None):
        """Unmap the peers' buffers, wait for everybody, then free the own one."""
        if self.local is None:
            return
        for r, p in enumerate(self.pointers):
            if r != self.rank:
                self._gw.lib.gw_ipc_close(p)
        torch.cuda.synchronize()
        dist.barrier(group=group)
        self._gw.lib.gw_ipc_free(self.local)
        self.local = None


class PeerMemoryExpertParallelMoe:
    """The expert-parallel layer with the exchange fused into the kernels on
    either side of it.  Instead of gather -> all-to-all -> regroup, the dispatch
    kernel quantises each routed row to NVFP4 with its expert's input scale and
    stores the 1584-byte record (1408 B of E2M1 + 176 scale bytes, against 5632 B
    of BF16) directly into the owning GPU's memory over NVLink, already at its
    expert-major position; the owner's grouped GEMMs read the records in place;
    the combine kernel reads each token's eight result rows from their owners'
    memory and folds them in expert order.  The 128-integer histograms and the
    two barriers of a step go through mailboxes in peer memory as well
    (gw_moe_ep_exchange); `exchange="nccl"` uses an all-gather and two all-reduces
    instead.

    Needs experts whose gate and up projections share their input scale (one
    quantised copy of a row serves both), as the fused checkpoint tensors do.
    """

    STAGES = ("route", "counts", "dispatch", "barrier_1", "experts", "barrier_2", "combine")
    RECORD_BYTES = 1584

    def __init__(self, experts_by_position, input_scales, rank: int, world: int, local_tokens: int,
                 receive_capacity_rows: int, placement: Placement | None = None, group=None,
                 send_home: bool = False, exchange: str = "peer", home_down=None):
        """experts_by_position: 128 entries indexed by physical position, None for
        experts of other ranks.  input_scales: the gate/up input scale of all 128
        experts by expert id (every rank quantises rows for every expert).
        send_home: the down GEMM's epilogue stores each result row into its source
        rank's memory and the source folds local rows; otherwise (default, faster
        in every measured configuration: the remote stores slow the GEMM down more
        than the pull costs) results stay with the owner and the combine kernel
        pulls them over NVLink.
        home_down: the down matrices of ALL 128 experts by expert id.  With them the owners run gate/up +
        GeGLU + quantisation only, every rank fetches the 416-byte quantised activations of its own rows
        (instead of 5632-byte BF16 results) and runs the down projection and the fold itself: the same
        bits, 14 times fewer bytes on the way back, a third of the expert weights on every rank."""
        import gewell_b200 as gw
        self.gw = gw
        self.placement = placement or Placement.contiguous(world)
        self.rank, self.world, self.group = rank, world, group
        self.per_rank = EXPERTS // world
        self.local_tokens, self.capacity = local_tokens, receive_capacity_rows
        self.table = gw.ExpertTable(experts_by_position)
        self.route_ws = gw.MoeWorkspace(local_tokens)
        self.expert_ws = gw.MoeWorkspace((receive_capacity_rows + 7) // 8)
        self.device = self.route_ws.device
        self.records = SharedBuffer(receive_capacity_rows * self.RECORD_BYTES, rank, world, group)
        self.send_home = send_home and world <= 8 and home_down is None
        self.home_table = None
        if home_down is not None:
            if len(home_down) != EXPERTS:
                raise ValueError("home_down needs the down matrices of all 128 experts")
            self.home_table = gw.ExpertTable([(None, None, down) for down in home_down])
            self.activation_records = SharedBuffer(
                receive_capacity_rows * int(gw.lib.gw_moe_ep_activation_record_bytes()), rank, world, group)
            self.returned = self.down = None
        elif self.send_home:
            self.returned = SharedBuffer(TOPK * local_tokens * HIDDEN * 2, rank, world, group)
            self.down = None
        else:
            self.returned = None
            self.down = SharedBuffer(receive_capacity_rows * HIDDEN * 2, rank, world, group)
        self.segment_start = torch.zeros(world * self.per_rank, dtype=torch.int32, device=self.device)
        self.home_base = torch.zeros(world * self.per_rank, dtype=torch.int32, device=self.device)
        scales = torch.tensor(list(input_scales), dtype=torch.float32)
        self.inverse_scales = (torch.ones_like(scales) / scales).to(self.device)      # IEEE FP32 division
        self.dest_rank = torch.tensor(self.placement.owner, dtype=torch.int32, device=self.device)
        self.physical = torch.tensor(self.placement.physical, dtype=torch.int32, device=self.device)
        self.counts_all = torch.zeros((world, EXPERTS), dtype=torch.int32, device=self.device)
        self.dest_row0 = torch.zeros(EXPERTS, dtype=torch.int32, device=self.device)
        self.local_offsets = torch.zeros(self.per_rank + 1, dtype=torch.int32, device=self.device)
        self.flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.timer = None
        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        self.exchange = exchange if world <= 8 else "nccl"
        self.mailbox = None
        if self.exchange == "peer":
            self.mailbox = SharedBuffer(int(gw.lib.gw_moe_ep_mailbox_bytes()), rank, world, group)
            torch.as_tensor(gw.ops._RawDeviceBytes(self.mailbox.local, self.mailbox.nbytes), device=self.device).zero_()
            self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize()
            dist.barrier(group=group)          # every mailbox is zero before the first flag arrives

    def _mark(self, name: str):
        if self.timer is not None:
            self.timer(name)

    def _barrier(self):
        # stream-ordered: completes on this rank only after every rank's earlier kernels have
        if self.exchange == "peer":
            self._exchange(None, 0, None)
        else:
            dist.all_reduce(self.flag, group=self.group)

    def _exchange(self, payload, count: int, gathered):
        self.gw.ops._check(self.gw.lib.gw_moe_ep_exchange(
            payload.data_ptr() if payload is not None else None, count, self.mailbox.pointer_table.data_ptr(), self.rank,
            self.world, self.epoch.data_ptr(), gathered.data_ptr() if gathered is not None else None,
            torch.cuda.current_stream().cuda_stream))

    def rows_received(self) -> int:
        """Rows this rank's experts processed in the last step (reads back one integer)."""
        return int(self.local_offsets[-1].item())

    def run(self, x, scores, expert_scales, rows: int, out=None):
        """One step; nothing is read back to the host, so the step can be
        enqueued ahead of the GPU (or captured)."""
        self.send(x, scores, expert_scales, rows)
        self.compute()
        return self.receive(rows, out)

    def send(self, x, scores, expert_scales, rows: int):
        """Routing, histogram exchange, destination tables, dispatch into the owners' memory."""
        lib, check = self.gw.lib, self.gw.ops._check
        stream = torch.cuda.current_stream().cuda_stream
        if rows > 0:
            self.route_ws.dispatch(scores, expert_scales, rows)
            offsets, _, _, _ = self.route_ws.routing_state(rows)
            counts = (offsets[1:] - offsets[:-1]).contiguous()
        else:                                  # a rank without tokens still serves its experts
            counts = torch.zeros(EXPERTS, dtype=torch.int32, device=self.device)
        self._mark("route")
        if self.exchange == "peer":
            self._exchange(counts, EXPERTS, self.counts_all)
        else:
            dist.all_gather_into_tensor(self.counts_all, counts, group=self.group)
        home = self.send_home
        check(lib.gw_moe_ep_tables(self.counts_all.data_ptr(), self.physical.data_ptr(), self.rank, self.world,
                                   self.dest_row0.data_ptr(), self.local_offsets.data_ptr(),
                                   self.segment_start.data_ptr() if home else None,
                                   self.home_base.data_ptr() if home else None, stream))
        self._mark("counts")
        if rows > 0:
            check(lib.gw_moe_ep_dispatch(self.route_ws._ws, x.data_ptr(), rows, self.inverse_scales.data_ptr(),
                                         self.dest_rank.data_ptr(), self.dest_row0.data_ptr(),
                                         self.records.pointer_table.data_ptr(), self.capacity, stream))
        self._mark("dispatch")
        self._barrier()
        self._mark("barrier_1")

    def compute(self, barrier: bool = True):
        """Grouped expert GEMMs over the records this rank received (and the barrier that
        tells every rank the results are ready)."""
        lib, check = self.gw.lib, self.gw.ops._check
        stream = torch.cuda.current_stream().cuda_stream
        home = self.send_home
        if self.home_table is not None:
            check(lib.gw_moe_ep_run_gate_up(self.expert_ws._ws, self.records.local, self.local_offsets.data_ptr(),
                                            self.rank * self.per_rank, self.per_rank, self.capacity, self.table.handle,
                                            self.activation_records.local, stream))
            self._mark("experts")
            if barrier:
                self.results_barrier()
            return
        check(lib.gw_moe_ep_run_experts(self.expert_ws._ws, self.records.local, self.local_offsets.data_ptr(),
                                        self.rank * self.per_rank, self.per_rank, self.capacity, self.table.handle,
                                        None if home else self.down.local,
                                        self.segment_start.data_ptr() if home else None,
                                        self.home_base.data_ptr() if home else None,
                                        self.returned.pointer_table.data_ptr() if home else None,
                                        TOPK * self.local_tokens, self.world, stream))
        self._mark("experts")
        if barrier:
            self.results_barrier()

    def results_barrier(self):
        self._barrier()
        self._mark("barrier_2")

    def receive(self, rows: int, out=None):
        """Ordered fold of each token's eight result rows (pulled from their owners, or local when sent home)."""
        lib, check = self.gw.lib, self.gw.ops._check
        stream = torch.cuda.current_stream().cuda_stream
        if out is None:
            out = torch.empty((rows, HIDDEN), dtype=torch.bfloat16, device=self.device)
        if rows == 0:
            pass
        elif self.home_table is not None:
            check(lib.gw_moe_ep_finish_at_home(self.route_ws._ws, rows, self.dest_rank.data_ptr(), self.dest_row0.data_ptr(),
                                               self.activation_records.pointer_table.data_ptr(), self.capacity,
                                               self.home_table.handle, out.data_ptr(), stream))
        elif self.send_home:
            _, _, inverse, weights = self.route_ws.routing_state(rows)
            check(lib.gw_moe_combine(self.returned.local, inverse.data_ptr(), weights.data_ptr(), rows, HIDDEN,
                                     out.data_ptr(), stream))
        else:
            check(lib.gw_moe_ep_combine(self.route_ws._ws, rows, self.dest_rank.data_ptr(), self.dest_row0.data_ptr(),
                                        self.down.pointer_table.data_ptr(), self.capacity, out.data_ptr(), stream))
        self._mark("combine")
        return out

    def close(self):
        self.records.close(self.group)
        for buffer in (self.down, self.returned, self.mailbox, getattr(self, "activation_records", None)):
            if buffer is not None:
                buffer.close(self.group)
