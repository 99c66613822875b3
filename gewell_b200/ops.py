"""Host-side mirror of the reference's operator interface over the C ABI.

Names and argument meaning follow the reference classes
(gewell::nvfp4::{Weight,Plan,dequantize}, gewell::fp8::{Weight,Plan},
sm120::{Projection,ExpertWeights,MoeWorkspace}); torch is used only for device
memory and the current stream.  Every call goes through libgewell_b200.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib

TRANSFORM_IDENTITY = _lib.TRANSFORM_IDENTITY
TRANSFORM_GELU_TANH_MULTIPLY = _lib.TRANSFORM_GELU_TANH_MULTIPLY


def _library():
    from . import lib
    return lib


def _ptr(t) -> int:
    if t is None:
        return 0
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream=None) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _check(status: int) -> None:
    _lib.check(_library(), status)


def kernel_error() -> int:
    """Error word written by the bounded waits of the tensor-core kernels
    (0 = none).  Synchronises the device and clears the word."""
    return int(_library().gw_debug_kernel_error())


def launch_count() -> int:
    """Kernels the CUDA library has launched in this process so far."""
    return int(_library().gw_debug_launch_count())


def rcp_approx(values):
    """rcp.approx.ftz.f32 of a NumPy float32 array, evaluated on the device
    (test aid: lets the CPU oracle use the hardware's reciprocal bits)."""
    import numpy as np
    flat = np.ascontiguousarray(values, dtype=np.float32)
    src = torch.from_numpy(flat.reshape(-1).copy()).cuda()
    dst = torch.empty_like(src)
    _check(_library().gw_debug_rcp_approx(_ptr(src), _ptr(dst), src.numel(), _stream()))
    return dst.cpu().numpy().reshape(flat.shape)


def geglu_bf16(gate, up):
    """Device GeGLU of BF16-valued NumPy float32 arrays (test aid, see rcp_approx)."""
    import numpy as np
    g = torch.from_numpy(np.ascontiguousarray(gate, dtype=np.float32)).to(torch.bfloat16).cuda()
    u = torch.from_numpy(np.ascontiguousarray(up, dtype=np.float32)).to(torch.bfloat16).cuda()
    out = torch.empty_like(g)
    _check(_library().gw_debug_geglu_bf16(_ptr(g), _ptr(u), _ptr(out), g.numel(), _stream()))
    return out.float().cpu().numpy()


# --------------------------------------------------------------------------- layout helpers

def nvfp4_scale_storage_bytes(rows: int, width: int) -> int:
    return int(_library().gw_nvfp4_scale_storage_bytes(rows, width))


def nvfp4_scale_offset(row: int, block: int, width: int) -> int:
    return int(_library().gw_nvfp4_scale_offset(row, block, width))


# --------------------------------------------------------------------------- NVFP4

@dataclass
class Nvfp4Weight:
    """gewell::nvfp4::Weight: packed [N,K/2] uint8 (even k low nibble), tiled
    E4M3 scales, FP32 dequantisation globals."""
    data: torch.Tensor
    scales: torch.Tensor
    input_scale: float
    weight_scale: float


def nvfp4_dequantize(weight: Nvfp4Weight, input_width: int, output_width: int, output=None, stream=None):
    """gewell::nvfp4::dequantize -> BF16 [N,K]."""
    if output is None:
        output = torch.empty((output_width, input_width), dtype=torch.bfloat16, device=weight.data.device)
    _check(_library().gw_nvfp4_dequantize(_ptr(weight.data), _ptr(weight.scales), weight.weight_scale,
                                          input_width, output_width, _ptr(output), _stream(stream)))
    return output


def absmax_bf16(values: torch.Tensor, stream=None):
    """(amax, nonfinite) of a BF16 tensor; reads the result back (synchronises)."""
    state = torch.zeros(2, dtype=torch.int32, device=values.device)
    _check(_library().gw_absmax_bf16(_ptr(values), values.numel(), _ptr(state), _stream(stream)))
    host = state.cpu()
    return host[:1].view(torch.float32).item(), bool(host[1].item())


def nvfp4_pack_weights(weights: torch.Tensor, input_scale: float = 1.0, weight_scale: float | None = None,
                       stream=None) -> Nvfp4Weight:
    """Device packer: BF16 [N,K] -> Nvfp4Weight (global = amax/(6*448) unless given)."""
    n, k = weights.shape
    if weight_scale is None:
        amax, bad = absmax_bf16(weights, stream)
        if bad:
            raise _lib.GewellInvalidArgument("NVFP4 source contains nonfinite weights")
        weight_scale = float(torch.tensor(amax / (6 * 448), dtype=torch.float64).to(torch.float32)) if amax else 1.0
    data = torch.empty((n, k // 2), dtype=torch.uint8, device=weights.device)
    scales = torch.empty(nvfp4_scale_storage_bytes(n, k), dtype=torch.uint8, device=weights.device)
    _check(_library().gw_nvfp4_pack_weights(_ptr(weights), n, k, weight_scale, _ptr(data), _ptr(scales), _stream(stream)))
    return Nvfp4Weight(data, scales, float(input_scale), float(weight_scale))


def nvfp4_quantize_activations(x: torch.Tensor, input_scale: float, width: int | None = None, gelu: bool = False,
                               stream=None):
    """Activation quantiser of nvfp4::Plan::run -> (packed [M,K/2], tiled scales)."""
    rows = x.shape[0]
    k = width if width is not None else (x.shape[1] // 2 if gelu else x.shape[1])
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty(nvfp4_scale_storage_bytes(rows, k), dtype=torch.uint8, device=x.device)
    _check(_library().gw_nvfp4_quantize_activations(
        _ptr(x), rows, k, input_scale, TRANSFORM_GELU_TANH_MULTIPLY if gelu else TRANSFORM_IDENTITY,
        _ptr(packed), _ptr(scales), _stream(stream)))
    return packed, scales


def nvfp4_gemv_w4a16(x: torch.Tensor, weight: Nvfp4Weight, input_width: int, output_width: int, stream=None):
    y = torch.empty((x.shape[0], output_width), dtype=torch.bfloat16, device=x.device)
    _check(_library().gw_nvfp4_gemv_w4a16(_ptr(x), x.shape[0], _ptr(weight.data), _ptr(weight.scales),
                                          weight.weight_scale, input_width, output_width, _ptr(y), _stream(stream)))
    return y


def nvfp4_linear_static_scratch(x, weight: Nvfp4Weight, input_width: int, output_width: int, y=None,
                                transform: int = TRANSFORM_IDENTITY, stream=None):
    """NVFP4 linear through the library's built-in scratch array: for callers
    that can neither allocate device memory nor spare a scratch buffer.  Takes
    inputs and outputs only; sizes above the built-in limit are rejected."""
    rows = x.shape[0]
    if y is None:
        y = torch.empty((rows, output_width), dtype=torch.bfloat16, device=x.device)
    _check(_library().gw_nvfp4_linear_static_scratch(_ptr(x), rows, input_width, output_width, _ptr(weight.data),
                                                     _ptr(weight.scales), weight.input_scale, weight.weight_scale,
                                                     _ptr(y), _stream(stream), transform))
    return y


class Nvfp4Plan:
    """gewell::nvfp4::Plan(handle, rows, K, N): scratch_bytes(), run(...)."""

    def __init__(self, rows: int, input_width: int, output_width: int):
        self._lib = _library()
        self._plan = ctypes.c_void_p()
        _check(self._lib.gw_nvfp4_plan_create(rows, input_width, output_width, ctypes.byref(self._plan)))
        self.rows, self.input_width, self.output_width = rows, input_width, output_width

    def scratch_bytes(self) -> int:
        return int(self._lib.gw_nvfp4_plan_scratch_bytes(self._plan))

    def run(self, x, weight: Nvfp4Weight, y, scratch, scratch_capacity=None, stream=None,
            transform: int = TRANSFORM_IDENTITY):
        capacity = scratch_capacity if scratch_capacity is not None else (
            scratch.numel() * scratch.element_size() if hasattr(scratch, "numel") else 0)
        _check(self._lib.gw_nvfp4_plan_run(self._plan, _ptr(x), _ptr(weight.data), _ptr(weight.scales),
                                           weight.input_scale, weight.weight_scale, _ptr(y), _ptr(scratch),
                                           capacity, _stream(stream), transform))
        return y

    def __del__(self):
        if getattr(self, "_plan", None):
            self._lib.gw_nvfp4_plan_destroy(self._plan)
            self._plan = None


# --------------------------------------------------------------------------- FP8

@dataclass
class Fp8Weight:
    """gewell::fp8::Weight: [N,K] E4M3FN codes, FP32 globals, optional
    per-output-channel alpha vector (input*weight scale) for joined projections."""
    data: torch.Tensor
    input_scale: float
    weight_scale: float
    channel_scales: torch.Tensor | None = None


def fp8_quantize_activations(x: torch.Tensor, input_scale: float, gelu: bool = False, stream=None):
    rows = x.shape[0]
    k = x.shape[1] // 2 if gelu else x.shape[1]
    packed = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    _check(_library().gw_fp8_quantize_activations(
        _ptr(x), rows, k, input_scale, TRANSFORM_GELU_TANH_MULTIPLY if gelu else TRANSFORM_IDENTITY,
        _ptr(packed), _stream(stream)))
    return packed


def fp8_pack_weights(weights: torch.Tensor, weight_scale: float = 0.0, row_scales: torch.Tensor | None = None,
                     stream=None) -> torch.Tensor:
    n, k = weights.shape
    data = torch.empty((n, k), dtype=torch.uint8, device=weights.device)
    _check(_library().gw_fp8_pack_weights(_ptr(weights), n, k, weight_scale, _ptr(row_scales), _ptr(data),
                                          _stream(stream)))
    return data


class Fp8Plan:
    """gewell::fp8::Plan(handle, rows, K, N, channel_scales)."""

    def __init__(self, rows: int, input_width: int, output_width: int, channel_scales: bool = False):
        self._lib = _library()
        self._plan = ctypes.c_void_p()
        _check(self._lib.gw_fp8_plan_create(rows, input_width, output_width, int(channel_scales),
                                            ctypes.byref(self._plan)))
        self.rows, self.input_width, self.output_width = rows, input_width, output_width

    def scratch_bytes(self) -> int:
        return int(self._lib.gw_fp8_plan_scratch_bytes(self._plan))

    def run(self, x, weight: Fp8Weight, y, scratch, scratch_capacity=None, stream=None,
            transform: int = TRANSFORM_IDENTITY):
        capacity = scratch_capacity if scratch_capacity is not None else (
            scratch.numel() * scratch.element_size() if hasattr(scratch, "numel") else 0)
        _check(self._lib.gw_fp8_plan_run(self._plan, _ptr(x), _ptr(weight.data), weight.input_scale,
                                         weight.weight_scale, _ptr(weight.channel_scales), _ptr(y), _ptr(scratch),
                                         capacity, _stream(stream), transform))
        return y

    def __del__(self):
        if getattr(self, "_plan", None):
            self._lib.gw_fp8_plan_destroy(self._plan)
            self._plan = None


# --------------------------------------------------------------------------- BF16

class Bf16Plan:
    """BF16 linear layer Y = X . W^T (the reference's BF16 LinearPlan / cublasGemmEx path)."""

    def __init__(self, rows: int, input_width: int, output_width: int):
        self._lib = _library()
        self._plan = ctypes.c_void_p()
        _check(self._lib.gw_bf16_plan_create(rows, input_width, output_width, ctypes.byref(self._plan)))
        self.rows, self.input_width, self.output_width = rows, input_width, output_width

    def scratch_bytes(self) -> int:
        return int(self._lib.gw_bf16_plan_scratch_bytes(self._plan))

    def run(self, x, weight, y, scratch=None, stream=None):
        capacity = scratch.numel() * scratch.element_size() if scratch is not None else 0
        _check(self._lib.gw_bf16_plan_run(self._plan, _ptr(x), _ptr(weight), _ptr(y), _ptr(scratch), capacity,
                                          _stream(stream)))
        return y

    def __del__(self):
        if getattr(self, "_plan", None):
            self._lib.gw_bf16_plan_destroy(self._plan)
            self._plan = None


# --------------------------------------------------------------------------- 26B projections

def bind_projection(storage: int, rows: int, columns: int, host_payload: bytes, device_payload: torch.Tensor):
    """sm120::bind_projection: describe one artifact entry (payload = weights [, tiled scales], two FP32
    globals at the end) as a Projection.  `device_payload` holds the same bytes on the device."""
    projection = _lib.Projection()
    buffer = (ctypes.c_uint8 * len(host_payload)).from_buffer_copy(host_payload)
    _check(_library().gw_bind_projection(storage, rows, columns, buffer, device_payload.data_ptr(), len(host_payload),
                                         ctypes.byref(projection)))
    return projection


class ProjectionWorkspace:
    """sm120::ProjectionWorkspace(projections, max_rows, policy, stream): prepare(rows, phase), run(...)."""

    def __init__(self, projections, max_rows: int, policy: int, stream=None):
        self._lib = _library()
        self._ws = ctypes.c_void_p()
        array = (_lib.Projection * len(projections))(*projections)
        _check(self._lib.gw_projection_workspace_create(array, len(projections), max_rows, policy, _stream(stream),
                                                        ctypes.byref(self._ws)))

    def prepare(self, rows: int, phase: int):
        _check(self._lib.gw_projection_workspace_prepare(self._ws, rows, phase))

    def run(self, projection, x, y):
        _check(self._lib.gw_projection_workspace_run(self._ws, ctypes.byref(projection), _ptr(x), _ptr(y)))
        return y

    def bytes(self) -> int:
        return int(self._lib.gw_projection_workspace_bytes(self._ws))

    def __del__(self):
        if getattr(self, "_ws", None):
            self._lib.gw_projection_workspace_destroy(self._ws)
            self._ws = None


class MlpChain:
    """31B Executor::project_mlp: gate + up projection -> GeGLU -> down projection of one layer from its
    three bound projections (make_projection), choosing joined / fused forms where the layout allows."""

    def __init__(self, hidden: int, mlp: int, max_rows: int, policy: int):
        self._lib = _library()
        self._chain = ctypes.c_void_p()
        self.hidden, self.mlp = hidden, mlp
        _check(self._lib.gw_mlp_chain_create(hidden, mlp, max_rows, policy, ctypes.byref(self._chain)))

    def prepare(self, rows: int):
        _check(self._lib.gw_mlp_chain_prepare(self._chain, rows))
        self.rows = rows

    def run(self, gate, up, down, x, phase: int, stream=None):
        rows = self.rows
        gate_up = torch.empty((rows, 2 * self.mlp), dtype=torch.bfloat16, device=x.device)
        product = torch.empty((rows, self.mlp), dtype=torch.bfloat16, device=x.device)
        y = torch.empty((rows, self.hidden), dtype=torch.bfloat16, device=x.device)
        _check(self._lib.gw_mlp_chain_run(self._chain, ctypes.byref(gate), ctypes.byref(up), ctypes.byref(down), _ptr(x),
                                          _ptr(gate_up), _ptr(product), _ptr(y), phase, _stream(stream)))
        return y

    def bytes(self) -> int:
        return int(self._lib.gw_mlp_chain_bytes(self._chain))

    def __del__(self):
        if getattr(self, "_chain", None):
            self._lib.gw_mlp_chain_destroy(self._chain)
            self._chain = None


class QkvProjector:
    """31B Executor::project_qkv without its norms: Q, K (and V) of one layer from their bound projections,
    as one joined GEMM where the weights lie back to back."""

    def __init__(self, hidden: int, q_width: int, kv_width: int, max_rows: int, policy: int):
        self._lib = _library()
        self._projector = ctypes.c_void_p()
        self.hidden, self.q, self.kv = hidden, q_width, kv_width
        _check(self._lib.gw_qkv_projector_create(hidden, q_width, kv_width, max_rows, policy, ctypes.byref(self._projector)))
        self.rows = 0

    def prepare(self, rows: int):
        _check(self._lib.gw_qkv_projector_prepare(self._projector, rows))
        self.rows = rows

    def run(self, query, key, value, x, phase: int, stream=None):
        """Returns (q, k, v) views ([rows, width] each; v None when `value` is None) and whether one joined GEMM ran."""
        rows, n = self.rows, self.q + self.kv * (2 if value is not None else 1)
        out = torch.empty((rows * n,), dtype=torch.bfloat16, device=x.device)
        q, k = out[:rows * self.q], out[rows * self.q:rows * (self.q + self.kv)]
        v = out[rows * (self.q + self.kv):] if value is not None else None
        joined = ctypes.c_int(0)
        _check(self._lib.gw_qkv_projector_run(self._projector, ctypes.byref(query), ctypes.byref(key),
                                              ctypes.byref(value) if value is not None else None, _ptr(x), _ptr(q), _ptr(k),
                                              _ptr(v), phase, _stream(stream), ctypes.byref(joined)))
        if joined.value:
            both = out.view(rows, n)
            return both[:, :self.q], both[:, self.q:self.q + self.kv], (both[:, self.q + self.kv:] if value is not None else None), True
        return q.view(rows, self.q), k.view(rows, self.kv), (v.view(rows, self.kv) if v is not None else None), False

    def bytes(self) -> int:
        return int(self._lib.gw_qkv_projector_bytes(self._projector))

    def __del__(self):
        if getattr(self, "_projector", None):
            self._lib.gw_qkv_projector_destroy(self._projector)
            self._projector = None


def join_nvfp4_pair(first, second, stream=None) -> bool:
    """In-place join of two bound NVFP4 projections (gw_join_nvfp4_pair); updates their pointers."""
    packed = first.physical_output * first.input // 2
    temp = torch.empty(2 * (packed + nvfp4_scale_storage_bytes(first.physical_output, first.input)), dtype=torch.uint8, device="cuda")
    joined = ctypes.c_int(0)
    _check(_library().gw_join_nvfp4_pair(ctypes.byref(first), ctypes.byref(second), _ptr(temp), temp.numel(), _stream(stream),
                                         ctypes.byref(joined)))
    torch.cuda.synchronize()
    return bool(joined.value)


def join_fp8_group(group, channel_scales: torch.Tensor, stream=None) -> bool:
    """In-place join of bound FP8 projections (gw_join_fp8_group); `group` is a ctypes array of Projection."""
    temp = torch.empty(sum(p.output * p.input for p in group), dtype=torch.uint8, device="cuda")
    joined = ctypes.c_int(0)
    _check(_library().gw_join_fp8_group(group, len(group), _ptr(channel_scales), _ptr(temp), temp.numel(), _stream(stream),
                                        ctypes.byref(joined)))
    return bool(joined.value)


# --------------------------------------------------------------------------- weight QDQ

def weight_qdq_apply(kind: int, values: torch.Tensor, stream=None) -> torch.Tensor:
    """weight_qdq::detail::apply_tensor: in-place fake quantisation (synchronises)."""
    state = torch.zeros(2, dtype=torch.int32, device=values.device)
    _check(_library().gw_weight_qdq_apply(kind, _ptr(values), values.numel(), _ptr(state), _stream(stream)))
    return values


# --------------------------------------------------------------------------- MoE

def make_projection(weight, input_width: int, output_width: int) -> _lib.Projection:
    """sm120::Projection (bind_projection, projection.cu:31-50) for an expert matrix: an Nvfp4Weight
    whose rows are already padded to a multiple of 128, an Fp8Weight, or a BF16 tensor [N, K]."""
    p = _lib.Projection()
    p.input, p.output = input_width, output_width
    p.physical_output = output_width
    if isinstance(weight, Nvfp4Weight):
        p.storage = _lib.STORAGE_NVFP4_W4A4
        p.physical_output = (output_width + 127) // 128 * 128
        p.nvfp4_data, p.nvfp4_scales = weight.data.data_ptr(), weight.scales.data_ptr()
        p.nvfp4_input_scale, p.nvfp4_weight_scale = weight.input_scale, weight.weight_scale
    elif isinstance(weight, Fp8Weight):
        p.storage = _lib.STORAGE_FP8_W8A8
        p.fp8_data = weight.data.data_ptr()
        p.fp8_input_scale, p.fp8_weight_scale = weight.input_scale, weight.weight_scale
        p.fp8_channel_scales = _ptr(weight.channel_scales) or None
    else:
        p.storage = _lib.STORAGE_BF16
        p.bf16 = weight.data_ptr()
    return p


class _RawDeviceBytes:
    """Zero-copy view of device memory through the CUDA array interface."""

    def __init__(self, pointer: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(pointer), False),
                                         "version": 2}


class ExpertTable:
    """The 128-entry ExpertWeights table, bound once (keeps the tensors alive)."""

    def __init__(self, experts: list[tuple | None]):
        """experts[i] = (gate, up, down), each an Nvfp4Weight, an Fp8Weight or a BF16 tensor [N, K];
        `experts[i] is None` marks an expert whose weights live on another rank (expert parallelism):
        no row may be routed to it on this rank.  A single projection may be None as well (a table that
        holds only the down matrices, for ranks that finish their own tokens' rows at home)."""
        self._lib = _library()
        self._keep = experts
        array = (_lib.ExpertWeights * len(experts))()
        for i, entry in enumerate(experts):
            if entry is None:
                array[i].gate.storage = array[i].up.storage = array[i].down.storage = _lib.STORAGE_ABSENT
                continue
            gate, up, down = entry
            for slot, weight, k, n in (("gate", gate, 2816, 704), ("up", up, 2816, 704), ("down", down, 704, 2816)):
                if weight is None:             # this projection is kept elsewhere
                    getattr(array[i], slot).storage = _lib.STORAGE_ABSENT
                else:
                    setattr(array[i], slot, make_projection(weight, k, n))
        self._table = ctypes.c_void_p()
        _check(self._lib.gw_moe_expert_table_create(array, len(experts), ctypes.byref(self._table)))

    @property
    def handle(self):
        return self._table

    def enable_w4a16(self, stream=None):
        """Make the BF16 copies that NVFP4 experts need to run with BF16 activations (set-up time)."""
        _check(self._lib.gw_moe_expert_table_enable_w4a16(self._table, _stream(stream)))

    def __del__(self):
        if getattr(self, "_table", None):
            self._lib.gw_moe_expert_table_destroy(self._table)
            self._table = None


class MoeWorkspace:
    """sm120::MoeWorkspace(max_rows): run, dispatch and the capture accessors."""

    def __init__(self, max_rows: int, device=None, fp8_experts: bool = False):
        self._lib = _library()
        self._ws = ctypes.c_void_p()
        self.max_rows = max_rows
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        _check(self._lib.gw_moe_create_ex(max_rows, 1 if fp8_experts else 0, ctypes.byref(self._ws)))
        self.rows = 0

    def dispatch(self, scores, expert_scales, rows: int, stream=None):
        _check(self._lib.gw_moe_dispatch(self._ws, _ptr(scores), _ptr(expert_scales), rows, _stream(stream)))
        self.rows = rows

    def run(self, x, scores, expert_scales, table: ExpertTable, y, rows: int, has_bf16=False, has_fp8=False,
            has_nvfp4=True, fp4=True, stream=None):
        _check(self._lib.gw_moe_run(self._ws, _ptr(x), _ptr(scores), _ptr(expert_scales), table.handle, _ptr(y), rows,
                                    int(has_bf16), int(has_fp8), int(has_nvfp4), int(fp4), _stream(stream)))
        self.rows = rows
        return y

    def run_sorted(self, x, offsets, first_expert: int, expert_count: int, total_rows: int, table: ExpertTable, y,
                   row_index=None, stream=None):
        """Expert MLP over rows sorted by local expert; sorted row i is
        x[row_index[i]] (x[i] when row_index is None)."""
        _check(self._lib.gw_moe_run_sorted(self._ws, _ptr(x), _ptr(row_index), _ptr(offsets), first_expert,
                                           expert_count, total_rows, table.handle, _ptr(y), _stream(stream)))
        return y

    def _alias(self, pointer: int, shape, dtype):
        """Zero-copy tensor over a workspace buffer (valid while the workspace lives)."""
        count = 1
        for s in shape:
            count *= s
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        raw = torch.as_tensor(_RawDeviceBytes(pointer, nbytes), device=self.device)
        return raw.view(dtype).reshape(shape)

    def routing_state(self, rows: int):
        """Aliases (no copies) of the routing results of the last dispatch over
        `rows` tokens: offsets [129], sorted_assignments [8*rows], inverse
        [8*rows], weights [8*rows]."""
        cached = getattr(self, "_routing_aliases", None)
        if cached is not None and cached[0] == rows:
            return cached[1]
        n = 8 * rows
        state = (self._alias(self._lib.gw_moe_offsets(self._ws), (129,), torch.int32),
                self._alias(self._lib.gw_moe_sorted_assignments(self._ws), (n,), torch.int32),
                self._alias(self._lib.gw_moe_inverse(self._ws), (n,), torch.int32),
                self._alias(self._lib.gw_moe_routing_weights(self._ws), (n,), torch.float32))
        self._routing_aliases = (rows, state)      # the buffers never move: build the views once per row count
        return state

    def _view(self, pointer: int, shape, dtype):
        """Copy of a workspace buffer as a tensor (the workspace owns the memory)."""
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype, device=self.device)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        raw = torch.as_tensor(_RawDeviceBytes(pointer, nbytes), device=self.device)
        return raw.view(dtype).reshape(shape).clone()

    def selected_experts(self):
        return self._view(self._lib.gw_moe_selected_experts(self._ws), (self.rows, 8), torch.int32)

    def routing_weights(self):
        return self._view(self._lib.gw_moe_routing_weights(self._ws), (self.rows, 8), torch.float32)

    def offsets(self):
        return self._view(self._lib.gw_moe_offsets(self._ws), (129,), torch.int32)

    def sorted_assignments(self):
        return self._view(self._lib.gw_moe_sorted_assignments(self._ws), (8 * self.rows,), torch.int32)

    def gate_up_capture(self):
        return self._view(self._lib.gw_moe_gate_up_capture(self._ws), (8 * self.rows, 1408), torch.bfloat16)

    def activated_capture(self):
        return self._view(self._lib.gw_moe_activated_capture(self._ws), (8 * self.rows, 704), torch.bfloat16)

    def down_capture(self):
        return self._view(self._lib.gw_moe_down_capture(self._ws), (8 * self.rows, 2816), torch.bfloat16)

    def quantized_input(self, parts: int = 1):
        """Test aid: copies of the quantised gate/up input of the last run: packed E2M1
        [parts, 8*rows, 1408] and the tiled scale storage [parts, scale_rows * 176]."""
        packed, scales = ctypes.c_void_p(), ctypes.c_void_p()
        scale_rows, part_rows = ctypes.c_uint32(), ctypes.c_uint32()
        _check(self._lib.gw_debug_moe_quantized_input(self._ws, ctypes.byref(packed), ctypes.byref(scales),
                                                      ctypes.byref(scale_rows), ctypes.byref(part_rows)))
        n = 8 * self.rows
        whole = self._alias(packed.value, (parts, part_rows.value, 1408), torch.uint8)
        tiles = self._alias(scales.value, (parts, scale_rows.value * 176), torch.uint8)
        return whole[:, :n].clone(), tiles.clone()

    def bytes(self) -> int:
        return int(self._lib.gw_moe_bytes(self._ws))

    STAGES = ("route_permute", "gather_quantise", "gate_up_gemm", "geglu_quantise", "down_gemm", "combine")

    def capture(self, enable: bool = True):
        """Also write the BF16 gate/up and activated intermediates when the fused path runs."""
        _check(self._lib.gw_moe_capture(self._ws, int(enable)))

    def stage_timing(self, enable: bool = True):
        _check(self._lib.gw_moe_stage_timing(self._ws, int(enable)))

    def stage_elapsed_ms(self) -> dict:
        out = (ctypes.c_float * 6)()
        _check(self._lib.gw_moe_stage_elapsed_ms(self._ws, out))
        return dict(zip(self.STAGES, [float(v) for v in out]))

    def __del__(self):
        if getattr(self, "_ws", None):
            self._lib.gw_moe_destroy(self._ws)
            self._ws = None


# --------------------------------------------------------------------------- 26B feed-forward block

def rsqrt_device(values):
    """rsqrtf evaluated on the device for a NumPy float32 array (test aid of the RMS norms)."""
    import numpy as np
    flat = np.ascontiguousarray(values, dtype=np.float32).ravel()
    out = np.empty_like(flat)
    _check(_library().gw_debug_rsqrt(flat.ctypes.data, out.ctypes.data, flat.size))
    return out.reshape(np.shape(values))


def rms_norm(x: torch.Tensor, weight=None, y=None, stream=None):
    """bf16_math::normalize over the rows of x [rows, width]."""
    y = torch.empty_like(x) if y is None else y
    _check(_library().gw_rms_norm_bf16(_ptr(x), _ptr(weight), _ptr(y), x.shape[0], x.shape[1], _stream(stream)))
    return y


def rms_norm_feedforward(x, shared_weight, router_weight, expert_weight, stream=None):
    """bf16_math::normalize_feedforward: (shared, router, expert) inputs from one RMS of x."""
    shared, router, expert = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
    _check(_library().gw_rms_norm_feedforward_bf16(_ptr(x), _ptr(shared_weight), _ptr(router_weight), _ptr(expert_weight),
                                                   _ptr(shared), _ptr(router), _ptr(expert), x.shape[0], x.shape[1],
                                                   _stream(stream)))
    return shared, router, expert


def add_bf16(a, b, y=None, stream=None):
    y = torch.empty_like(a) if y is None else y
    _check(_library().gw_add_bf16(_ptr(a), _ptr(b), _ptr(y), a.numel(), _stream(stream)))
    return y


def scale_bf16(x, scalar, stream=None):
    """x *= scalar[0] in place (row_scale of the 26B executor)."""
    _check(_library().gw_scale_bf16(_ptr(x), _ptr(scalar), x.numel(), _stream(stream)))
    return x


def ffn_tail(shared_mlp, routed, norm_shared, norm_routed, norm_sum, layer_scalar, hidden, stream=None):
    """Post norms, adds and the layer scalar of the block in one launch; updates hidden in place."""
    _check(_library().gw_ffn_tail_bf16(_ptr(shared_mlp), _ptr(routed), _ptr(norm_shared), _ptr(norm_routed), _ptr(norm_sum),
                                       _ptr(layer_scalar), _ptr(hidden), hidden.shape[0], hidden.shape[1], _stream(stream)))
    return hidden


class FfnBlock:
    """The feed-forward block of 26B layers (shared MLP + router + MoE + norms and residuals).

    layers: list of dicts with the BF16 tensors pre_feedforward_norm, router_scale, pre_feedforward_norm_2,
    post_feedforward_norm_1, post_feedforward_norm_2, post_feedforward_norm, layer_scalar, router_proj,
    router_per_expert_scale, the shared-MLP weights gate / up / down (Nvfp4Weight, Fp8Weight or BF16 tensor)
    and `experts` (an ExpertTable), plus optional has_bf16 / has_fp8 / has_nvfp4 flags."""

    BUFFERS = {"normalized": (0, 2816), "router_input": (1, 2816), "expert_input": (2, 2816), "shared_mlp": (3, 2816),
               "router_logits": (4, 128), "routed": (5, 2816)}

    def __init__(self, layers, max_rows: int, policy: int, fp8_experts: bool = False, stream=None):
        self._lib = _library()
        self._keep = layers
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._weights = (_lib.FfnBlockWeights * len(layers))()
        for w, layer in zip(self._weights, layers):
            for name in ("pre_feedforward_norm", "router_scale", "pre_feedforward_norm_2", "post_feedforward_norm_1",
                         "post_feedforward_norm_2", "post_feedforward_norm", "layer_scalar", "router_proj",
                         "router_per_expert_scale"):
                setattr(w, name, _ptr(layer[name]))
            w.gate = make_projection(layer["gate"], 2816, 2112)
            w.up = make_projection(layer["up"], 2816, 2112)
            w.down = make_projection(layer["down"], 2112, 2816)
            w.experts = layer["experts"].handle
            w.has_bf16 = int(layer.get("has_bf16", False))
            w.has_fp8 = int(layer.get("has_fp8", False))
            w.has_nvfp4 = int(layer.get("has_nvfp4", True))
        self._block = ctypes.c_void_p()
        _check(self._lib.gw_ffn_block_create(self._weights, len(layers), max_rows, policy, 1 if fp8_experts else 0,
                                             _stream(stream), ctypes.byref(self._block)))
        self.rows = 0

    def prepare(self, rows: int, phase: int):
        _check(self._lib.gw_ffn_block_prepare(self._block, rows, phase))
        self.rows = rows

    def run(self, layer: int, hidden: torch.Tensor):
        """Applies layer `layer`'s block to hidden [rows, 2816] in place."""
        _check(self._lib.gw_ffn_block_run(self._block, ctypes.byref(self._weights[layer]), _ptr(hidden)))
        return hidden

    def buffer(self, name: str) -> torch.Tensor:
        """Copy of an intermediate of the last run."""
        which, width = self.BUFFERS[name]
        pointer = self._lib.gw_ffn_block_buffer(self._block, which)
        raw = torch.as_tensor(_RawDeviceBytes(pointer, self.rows * width * 2), device=self.device)
        return raw.view(torch.bfloat16).reshape(self.rows, width).clone()

    def selected_experts(self) -> torch.Tensor:
        pointer = self._lib.gw_moe_selected_experts(self._lib.gw_ffn_block_moe(self._block))
        raw = torch.as_tensor(_RawDeviceBytes(pointer, self.rows * 8 * 4), device=self.device)
        return raw.view(torch.int32).reshape(self.rows, 8).clone()

    def bytes(self) -> int:
        return int(self._lib.gw_ffn_block_bytes(self._block))

    def __del__(self):
        if getattr(self, "_block", None):
            self._lib.gw_ffn_block_destroy(self._block)
            self._block = None


def gather_rows(x, index, divisor: int, rows: int, stream=None):
    out = torch.empty((rows, x.shape[1]), dtype=torch.bfloat16, device=x.device)
    _check(_library().gw_gather_rows_bf16(_ptr(x), _ptr(index), divisor, rows, x.shape[1], _ptr(out), _stream(stream)))
    return out


def moe_combine(down, inverse, weights, rows: int, stream=None):
    out = torch.empty((rows, down.shape[1]), dtype=torch.bfloat16, device=down.device)
    _check(_library().gw_moe_combine(_ptr(down), _ptr(inverse), _ptr(weights), rows, down.shape[1], _ptr(out),
                                     _stream(stream)))
    return out
