"""Host-side mirror of forja's backend interface over the C ABI of libforja_cuda.so.

Names and semantics follow ``forja_core`` (crates/forja-core/src/backend.rs:650-984, ops.rs:163-302,
layout.rs): ``CudaBackend.alloc/view/write/read/release/submit``, ``Tensor`` + ``Layout`` views,
``CommandList.dispatch`` with the reference's operand orders, ``Submission.wait``. This module is a
test and benchmark harness; the product is the library behind it. There is no CPU path: creating a
backend without a CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _lib

F32, F16, BF16, I32, U32 = 0, 1, 2, 3, 4
DTYPE_SIZE = {F32: 4, F16: 2, BF16: 2, I32: 4, U32: 4}
NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16, I32: np.int32, U32: np.uint32}

STATUS_NAMES = ["Ok", "QuotaExceeded", "AllocationFailed", "ExecutionFailed", "DeviceExecutionFailed", "DeviceErrorFlag",
                "Timeout", "InvalidInput", "UnsupportedOperation", "IndexOutOfRange"]
OK, QUOTA_EXCEEDED, ALLOCATION_FAILED, EXECUTION_FAILED, DEVICE_EXECUTION_FAILED, DEVICE_ERROR_FLAG, TIMEOUT, INVALID_INPUT, \
    UNSUPPORTED_OPERATION, INDEX_OUT_OF_RANGE = range(10)
POOL_SHARED_TAIL, POOL_INVALID_CHECKPOINT, POOL_CORRUPT_STATE = 30, 31, 32


class BackendError(RuntimeError):
    """forja_core::BackendError (crates/forja-core/src/backend.rs:362-426)."""

    def __init__(self, status: int, index: Optional[int] = None, dispatch: Optional[int] = None, flag: Optional[int] = None):
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"BackendError::{name}" + (f" index={index}" if index is not None else ""))
        self.status, self.index, self.dispatch, self.flag = status, index, dispatch, flag


def _check(status: int):
    if status != OK:
        raise BackendError(status)


@dataclass(frozen=True)
class Layout:
    """Strided view metadata in elements (crates/forja-core/src/layout.rs)."""
    dtype: int
    offset: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]

    @staticmethod
    def contiguous(dtype: int, shape: Sequence[int], offset: int = 0) -> "Layout":
        strides, acc = [], 1
        for extent in reversed(shape):
            strides.append(acc)
            acc *= extent
        return Layout(dtype, offset, tuple(shape), tuple(reversed(strides)))

    def element_count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def is_contiguous(self) -> bool:
        return self.strides == Layout.contiguous(self.dtype, self.shape).strides or self.element_count() <= 1

    def slice(self, specs: Sequence[Tuple[int, int, int]]) -> "Layout":
        """specs: (start, len, step) per axis, like ViewOp::Slice."""
        if len(specs) != len(self.shape):
            raise BackendError(INVALID_INPUT)
        offset, shape, strides = self.offset, [], []
        for (start, length, step), extent, stride in zip(specs, self.shape, self.strides):
            if step == 0 or (length and start + (length - 1) * step >= extent):
                raise BackendError(INVALID_INPUT)
            offset += start * stride
            shape.append(length)
            strides.append(stride * step)
        return Layout(self.dtype, offset, tuple(shape), tuple(strides))

    def reshape(self, shape: Sequence[int]) -> "Layout":
        if not self.is_contiguous():
            raise BackendError(INVALID_INPUT)
        new = Layout.contiguous(self.dtype, shape, self.offset)
        if new.element_count() != self.element_count():
            raise BackendError(INVALID_INPUT)
        return new

    def permute(self, axes: Sequence[int]) -> "Layout":
        if sorted(axes) != list(range(len(self.shape))):
            raise BackendError(INVALID_INPUT)
        return Layout(self.dtype, self.offset, tuple(self.shape[a] for a in axes), tuple(self.strides[a] for a in axes))

    def broadcast(self, shape: Sequence[int]) -> "Layout":
        if len(shape) < len(self.shape):
            raise BackendError(INVALID_INPUT)
        pad = len(shape) - len(self.shape)
        old_shape, old_strides = (1,) * pad + self.shape, (0,) * pad + self.strides
        strides = []
        for want, have, stride in zip(shape, old_shape, old_strides):
            if have == want:
                strides.append(stride)
            elif have == 1:
                strides.append(0)
            else:
                raise BackendError(INVALID_INPUT)
        return Layout(self.dtype, self.offset, tuple(shape), tuple(strides))


@dataclass(frozen=True)
class Tensor:
    """Validated view into a backend allocation (crates/forja-core/src/ops.rs:90-159)."""
    buffer: int
    layout: Layout
    byte_len: int
    writable: bool = True

    @property
    def shape(self):
        return self.layout.shape

    @property
    def dtype(self):
        return self.layout.dtype

    def slice(self, specs): return Tensor(self.buffer, self.layout.slice(specs), self.byte_len, self.writable)
    def reshape(self, shape): return Tensor(self.buffer, self.layout.reshape(shape), self.byte_len, self.writable)
    def permute(self, axes): return Tensor(self.buffer, self.layout.permute(axes), self.byte_len, self.writable)
    def broadcast(self, shape): return Tensor(self.buffer, self.layout.broadcast(shape), self.byte_len, self.writable)

    def narrow(self, axis: int, start: int, length: int) -> "Tensor":
        specs = [(0, s, 1) for s in self.shape]
        specs[axis] = (start, length, 1)
        return self.slice(specs)

    def to_c(self) -> _lib.FjTensor:
        t = _lib.FjTensor()
        t.buffer, t.dtype, t.rank, t.offset = self.buffer, self.layout.dtype, len(self.layout.shape), self.layout.offset
        for i, (s, st) in enumerate(zip(self.layout.shape, self.layout.strides)):
            t.shape[i], t.strides[i] = s, st
        return t


# fj_op codes (include/forja_cuda.h)
OP_PROGRAM, OP_COPY, OP_PAGED_COPY, OP_RMS_NORM, OP_ARGMAX, OP_TOP_K, OP_ROPE, OP_EMBED, OP_QUANT_EMBED, OP_MATMUL, OP_QUANT_MATMUL, \
    OP_GATHER_QUANT_MATMUL, OP_PAGED_SDPA, OP_PAGED_SDPA_APPEND, OP_SDPA, OP_SAMPLE, OP_GATHER_MATMUL = range(1, 18)


@dataclass(frozen=True)
class Op:
    """forja_core::Op (crates/forja-core/src/ops.rs:163-302) with its scalar parameters."""
    code: int
    u0: int = 0
    u1: int = 0
    u2: int = 0
    u3: int = 0
    f0: float = 0.0
    program: int = 0

    @staticmethod
    def Copy(): return Op(OP_COPY)
    @staticmethod
    def PagedCopy(into_pages: bool, start: int, page_tokens: int): return Op(OP_PAGED_COPY, u0=0 if into_pages else 1, u1=start, u2=page_tokens)
    @staticmethod
    def RmsNorm(eps: float): return Op(OP_RMS_NORM, f0=eps)
    @staticmethod
    def Argmax(chunk_width: int = 2048): return Op(OP_ARGMAX)
    @staticmethod
    def TopK(k: int, normalize: bool, chunk_width: int = 2048): return Op(OP_TOP_K, u0=k, u1=int(normalize))
    @staticmethod
    def Sample(position: int): return Op(OP_SAMPLE, u0=position)  # inputs [logits, params(5 x u32)] or, masked, [logits, params, allow]
    @staticmethod
    def Rope(theta: float): return Op(OP_ROPE, f0=theta)
    @staticmethod
    def Embed(): return Op(OP_EMBED)
    @staticmethod
    def QuantEmbed(bits: int, group_size: int): return Op(OP_QUANT_EMBED, u0=bits, u1=group_size)
    @staticmethod
    def Matmul(epilogue: int = 0): return Op(OP_MATMUL, program=epilogue)  # with an epilogue: inputs [a, b, extra]
    @staticmethod
    def QuantMatmul(bits: int, group_size: int, epilogue: int = 0): return Op(OP_QUANT_MATMUL, u0=bits, u1=group_size, program=epilogue)
    @staticmethod
    def GatherQuantMatmul(bits: int, group_size: int, epilogue: int = 0): return Op(OP_GATHER_QUANT_MATMUL, u0=bits, u1=group_size, program=epilogue)
    @staticmethod
    def PagedSdpa(scale: float, causal: bool, q_start: int, key_length: int, page_tokens: int):
        return Op(OP_PAGED_SDPA, u0=int(causal), u1=q_start, u2=key_length, u3=page_tokens, f0=scale)
    @staticmethod
    def PagedSdpaAppend(scale: float, q_start: int, page_tokens: int): return Op(OP_PAGED_SDPA_APPEND, u1=q_start, u3=page_tokens, f0=scale)
    @staticmethod
    def Sdpa(scale: float, causal: bool, q_start: int): return Op(OP_SDPA, u0=int(causal), u1=q_start, f0=scale)
    @staticmethod
    def GatherMatmul(): return Op(OP_GATHER_MATMUL)
    @staticmethod
    def Program(handle: int): return Op(OP_PROGRAM, program=handle)


@dataclass
class Dispatch:
    op: Op
    inputs: List[Tensor]
    outputs: List[Tensor]


@dataclass
class CommandList:
    """Ordered validated dispatches (crates/forja-core/src/ops.rs CommandList)."""
    dispatches: List[Dispatch] = field(default_factory=list)

    def dispatch(self, op: Op, inputs: Sequence[Tensor], output: Tensor):
        self.dispatches.append(Dispatch(op, list(inputs), [output]))
        return self

    def dispatch_many(self, op: Op, inputs: Sequence[Tensor], outputs: Sequence[Tensor]):
        self.dispatches.append(Dispatch(op, list(inputs), list(outputs)))
        return self


class Submission:
    """forja_core::Submission (crates/forja-core/src/backend.rs:609-647)."""

    def __init__(self, lib, handle, keepalive):
        self._lib, self._h, self._keep = lib, handle, keepalive

    def wait(self, timeout_ns: int = 0):
        status = self._lib.fj_sub_wait(self._h, timeout_ns)
        if status in (INDEX_OUT_OF_RANGE, DEVICE_ERROR_FLAG, DEVICE_EXECUTION_FAILED):
            err = _lib.FjDeviceError()
            self._lib.fj_sub_error(self._h, C.byref(err))
            raise BackendError(status, index=err.value, dispatch=err.dispatch, flag=err.flag)
        _check(status)

    def gpu_time_ns(self) -> int:
        out = C.c_uint64(0)
        _check(self._lib.fj_sub_gpu_time_ns(self._h, C.byref(out)))
        return out.value

    def completion_serial(self) -> int:
        return self._lib.fj_sub_completion_serial(self._h)

    def kernel_launches(self) -> int:
        return self._lib.fj_sub_kernel_launches(self._h)

    def profile(self):
        n = C.c_uint32(0)
        self._lib.fj_sub_profile(self._h, None, 0, C.byref(n))
        arr = (_lib.FjDispatchProfile * max(n.value, 1))()
        self._lib.fj_sub_profile(self._h, arr, n.value, C.byref(n))
        return [(arr[i].op, arr[i].kernels, arr[i].ns) for i in range(n.value)]

    def profile_costs(self):
        """Per dispatch {op, kernels, ns, read_bytes, write_bytes, flops}: device time beside the reference's KernelCost."""
        n = C.c_uint32(0)
        self._lib.fj_sub_profile(self._h, None, 0, C.byref(n))
        arr = (_lib.FjDispatchProfile * max(n.value, 1))()
        self._lib.fj_sub_profile(self._h, arr, n.value, C.byref(n))
        return [{"op": arr[i].op, "kernels": arr[i].kernels, "ns": arr[i].ns, "read_bytes": arr[i].read_bytes, "write_bytes": arr[i].write_bytes,
                 "flops": arr[i].flops} for i in range(n.value)]

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.fj_sub_destroy(self._h)
            self._h = None


GRAPH_FIELD_U0, GRAPH_FIELD_U1, GRAPH_FIELD_U2, GRAPH_FIELD_U3 = 0, 1, 2, 3
GRAPH_FIELD_INPUT_OFFSET, GRAPH_FIELD_OUTPUT_OFFSET, GRAPH_FIELD_INPUT_EXTENT, GRAPH_FIELD_OUTPUT_EXTENT = 0x100, 0x200, 0x300, 0x400


class PreparedGraph:
    """forja_core::PreparedGraph (crates/forja-core/src/graph.rs:1077-1160): a retained command template replayed with parameter values."""

    def __init__(self, lib, handle, n_params: int):
        self._lib, self._h, self.n_params = lib, handle, n_params

    def replay(self, values: Sequence[int], profiled: bool = False) -> Submission:
        raw = (C.c_uint32 * max(len(values), 1))(*values)
        handle = C.c_void_p()
        _check(self._lib.fj_graph_replay(self._h, raw, len(values), int(profiled), C.byref(handle)))
        return Submission(self._lib, handle, [])

    def close(self):
        if self._h:
            self._lib.fj_graph_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class CudaBackend:
    """The `forja-cuda` backend: one CUDA device, one stream, hand-written sm_100a kernels."""

    def __init__(self, device: int = 0, memory_limit: int = 0):
        self._lib = _lib.load()
        handle = C.c_void_p()
        status = self._lib.fj_backend_create(device, memory_limit, C.byref(handle))
        if status != OK:
            raise BackendError(status)
        self._h = handle
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            self._lib.fj_backend_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    # -- Backend trait ----------------------------------------------------------------------
    def device_info(self):
        info = _lib.FjDeviceInfo()
        _check(self._lib.fj_device_info(self._h, C.byref(info)))
        return {"name": info.name.decode(), "sm_count": info.sm_count, "cc": (info.cc_major, info.cc_minor),
                "total_memory": info.total_memory, "l2_bytes": info.l2_bytes, "max_smem_per_block": info.max_smem_per_block}

    def memory_usage(self):
        used, limit = C.c_uint64(0), C.c_uint64(0)
        _check(self._lib.fj_memory_usage(self._h, C.byref(used), C.byref(limit)))
        return used.value, limit.value

    def set_memory_limit(self, nbytes: int):
        _check(self._lib.fj_set_memory_limit(self._h, nbytes))

    def alloc(self, dtype: int, shape: Sequence[int]) -> Tensor:
        layout = Layout.contiguous(dtype, tuple(int(s) for s in shape))
        nbytes = layout.element_count() * DTYPE_SIZE[dtype]
        buf = C.c_uint64(0)
        _check(self._lib.fj_alloc(self._h, nbytes, C.byref(buf)))
        return Tensor(buf.value, layout, nbytes, True)

    def import_readonly(self, array: np.ndarray, dtype: int) -> Tensor:
        array = np.ascontiguousarray(array)
        buf = C.c_uint64(0)
        _check(self._lib.fj_import_readonly(self._h, array.ctypes.data_as(C.c_void_p), array.nbytes, C.byref(buf)))
        return Tensor(buf.value, Layout.contiguous(dtype, array.shape), array.nbytes, False)

    def view(self, tensor: Tensor, kind: str, arg) -> Tensor:
        return getattr(tensor, kind)(arg)

    def write(self, tensor: Tensor, data) -> None:
        if not tensor.writable or not tensor.layout.is_contiguous():
            raise BackendError(INVALID_INPUT)
        data = np.ascontiguousarray(data)
        if data.nbytes != tensor.layout.element_count() * DTYPE_SIZE[tensor.dtype]:
            raise BackendError(INVALID_INPUT)
        _check(self._lib.fj_write(self._h, tensor.buffer, tensor.layout.offset * DTYPE_SIZE[tensor.dtype], data.ctypes.data_as(C.c_void_p), data.nbytes))

    def read(self, tensor: Tensor) -> np.ndarray:
        out = np.empty(tensor.shape, NP_OF[tensor.dtype])
        if out.size == 0:
            return out
        t = tensor.to_c()
        _check(self._lib.fj_read_strided(self._h, C.byref(t), out.ctypes.data_as(C.c_void_p)))
        return out

    def release(self, tensor: Tensor) -> None:
        _check(self._lib.fj_release(self._h, tensor.buffer))

    def prepare_program(self, kind: int, insts: np.ndarray, outputs: np.ndarray) -> int:
        insts = np.ascontiguousarray(insts, np.uint32)
        outputs = np.ascontiguousarray(outputs, np.uint32)
        handle = C.c_uint64(0)
        _check(self._lib.fj_program_prepare(self._h, kind, insts.ctypes.data_as(C.c_void_p), insts.shape[0], outputs.ctypes.data_as(C.c_void_p), outputs.shape[0], C.byref(handle)))
        return handle.value

    def program_info(self, handle: int):
        kernel = C.c_uint32(0)
        consts = (C.c_float * 4)()
        _check(self._lib.fj_program_info(self._h, handle, C.byref(kernel), consts))
        return kernel.value, tuple(consts)

    @staticmethod
    def _encode(commands: CommandList):
        n = len(commands.dispatches)
        arr = (_lib.FjDispatch * max(n, 1))()
        keep = []
        for i, d in enumerate(commands.dispatches):
            ins = (_lib.FjTensor * max(len(d.inputs), 1))(*[t.to_c() for t in d.inputs])
            outs = (_lib.FjTensor * max(len(d.outputs), 1))(*[t.to_c() for t in d.outputs])
            keep += [ins, outs]
            arr[i].op, arr[i].n_inputs, arr[i].n_outputs = d.op.code, len(d.inputs), len(d.outputs)
            arr[i].u0, arr[i].u1, arr[i].u2, arr[i].u3, arr[i].f0, arr[i].program = d.op.u0, d.op.u1, d.op.u2, d.op.u3, d.op.f0, d.op.program
            arr[i].inputs, arr[i].outputs = ins, outs
        return arr, n, keep

    def submit(self, commands: CommandList, profiled: bool = False) -> Submission:
        arr, n, keep = self._encode(commands)
        handle = C.c_void_p()
        _check(self._lib.fj_submit(self._h, arr, n, int(profiled), C.byref(handle)))
        return Submission(self._lib, handle, keep)

    def prepare_graph(self, commands: CommandList, bindings: Sequence[Tuple[int, int, int, int, int]], n_params: int) -> "PreparedGraph":
        """Backend::prepare_graph: ``bindings`` are (dispatch, field code, parameter, scale, offset) with the field codes of
        include/forja_cuda.h (GRAPH_FIELD_*); the bound field becomes offset + scale * values[parameter] at every replay."""
        arr, n, _ = self._encode(commands)
        raw = (_lib.FjGraphBinding * max(len(bindings), 1))()
        for i, (dispatch, field_code, param, scale, offset) in enumerate(bindings):
            raw[i].dispatch, raw[i].field, raw[i].param, raw[i].scale, raw[i].offset = dispatch, field_code, param, scale, offset
        handle = C.c_void_p()
        _check(self._lib.fj_graph_prepare(self._h, arr, n, raw, len(bindings), n_params, C.byref(handle)))
        return PreparedGraph(self._lib, handle, n_params)

    # -- helpers for tests and benchmarks -----------------------------------------------------
    def tensor_from(self, array: np.ndarray, dtype: int) -> Tensor:
        t = self.alloc(dtype, array.shape)
        self.write(t, array)
        return t

    def run(self, op: Op, inputs: Sequence[Tensor], outputs: Sequence[Tensor]):
        cl = CommandList()
        cl.dispatch_many(op, inputs, outputs)
        sub = self.submit(cl)
        sub.wait()
        return sub

    def fill_random(self, tensor: Tensor, seed: int, mean: float = 0.0, std: float = 1.0):
        """Synthetic contents for a whole contiguous tensor (normal for floats, random words for u32)."""
        _check(self._lib.fj_fill_random(self._h, tensor.buffer, tensor.layout.offset * DTYPE_SIZE[tensor.dtype], tensor.layout.element_count(), tensor.dtype, seed, mean, std))

    def tcgen05_wait_giveups(self) -> int:
        out = C.c_uint32(0)
        _check(self._lib.fj_tcgen05_wait_giveups(self._h, C.byref(out)))
        return out.value

    def synchronize(self):
        _check(self._lib.fj_synchronize(self._h))

    def kernel_launch_count(self) -> int:
        return self._lib.fj_kernel_launch_count(self._h)

    def device_ptr(self, tensor: Tensor) -> int:
        """Device address of the first element of a tensor view."""
        ptr, size = C.c_void_p(), C.c_uint64(0)
        _check(self._lib.fj_buffer_device_ptr(self._h, tensor.buffer, C.byref(ptr), C.byref(size)))
        return (ptr.value or 0) + tensor.layout.offset * DTYPE_SIZE[tensor.dtype]

    def decode_attention_static(self, q: Tensor, out: Tensor, kpool: Tensor, vpool: Tensor, tables: Tensor, generations: Tensor,
                                key_lengths, scale: float, status: Optional[Tensor] = None) -> int:
        """fj_paged_decode_attention_static: decode attention whose scratch is a fixed array inside
        the library (no allocation). q/out [lanes, q_heads, 128]; tables [lanes, table_pages, 2].
        Returns the fj_status; FJ_QUOTA_EXCEEDED when the batch exceeds the array's limits."""
        lengths = np.ascontiguousarray(key_lengths, np.uint32)
        lanes, q_heads = q.shape[0], q.shape[1]
        return self._lib.fj_paged_decode_attention_static(
            self._h, self.device_ptr(q), self.device_ptr(out), self.device_ptr(kpool), self.device_ptr(vpool), self.device_ptr(tables),
            self.device_ptr(generations), lengths.ctypes.data_as(C.c_void_p), lanes, tables.shape[1], kpool.shape[0], q_heads, kpool.shape[2],
            q.dtype, scale, self.device_ptr(status) if status is not None else None)

    def timer(self) -> int:
        t = C.c_uint64(0)
        _check(self._lib.fj_timer_create(self._h, C.byref(t)))
        return t.value

    def timer_record(self, timer: int):
        _check(self._lib.fj_timer_record(self._h, timer))

    def timer_elapsed_ns(self, start: int, stop: int) -> int:
        out = C.c_uint64(0)
        _check(self._lib.fj_timer_elapsed_ns(self._h, start, stop, C.byref(out)))
        return out.value


class KvPool:
    """Device-resident paged-KV allocator and ragged-batch packer (fj_kvpool_*, fj_pack_step)."""

    def __init__(self, backend: CudaBackend, page_tokens: int, physical_pages: int, lanes: int, table_pages: int):
        self.backend, self._lib = backend, backend._lib
        self.page_tokens, self.physical_pages, self.lanes, self.table_pages = page_tokens, physical_pages, lanes, table_pages
        handle = C.c_void_p()
        _check(self._lib.fj_kvpool_create(backend._h, page_tokens, physical_pages, lanes, table_pages, C.byref(handle)))
        self._h = handle

    def close(self):
        if getattr(self, "_h", None) and getattr(self.backend, "_h", None):
            self._lib.fj_kvpool_destroy(self._h)
        self._h = None

    def reserve(self, lanes: Sequence[int], tokens: Sequence[int], want_status: bool = True):
        la, to = np.ascontiguousarray(lanes, np.uint32), np.ascontiguousarray(tokens, np.uint32)
        status = np.zeros(la.size, np.int32)
        _check(self._lib.fj_kvpool_reserve(self._h, la.ctypes.data_as(C.c_void_p), to.ctypes.data_as(C.c_void_p), la.size,
                                           status.ctypes.data_as(C.c_void_p) if want_status else None))
        return status.tolist() if want_status else None

    def release(self, lanes: Sequence[int]):
        la = np.ascontiguousarray(lanes, np.uint32)
        _check(self._lib.fj_kvpool_release(self._h, la.ctypes.data_as(C.c_void_p), la.size))

    def table(self, lane: int) -> np.ndarray:
        out = np.zeros((self.table_pages, 2), np.uint32)
        _check(self._lib.fj_kvpool_read_table(self._h, lane, out.ctypes.data_as(C.c_void_p)))
        return out

    def generations(self) -> np.ndarray:
        out = np.zeros(self.physical_pages, np.uint32)
        _check(self._lib.fj_kvpool_read_generations(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def free_list(self) -> np.ndarray:
        out = np.zeros(self.physical_pages, np.uint32)
        n = C.c_uint32(0)
        _check(self._lib.fj_kvpool_read_free(self._h, out.ctypes.data_as(C.c_void_p), self.physical_pages, C.byref(n)))
        return out[:n.value]

    def refcounts(self) -> np.ndarray:
        out = np.zeros(self.physical_pages, np.uint32)
        _check(self._lib.fj_kvpool_read_refcounts(self._h, out.ctypes.data_as(C.c_void_p)))
        return out

    def fork(self, src_lane: int, src_logical_len: int, dst_lane: int, prefix_tokens: int, reserved_tokens: int) -> int:
        """PagedSequence::fork_reserved on the device pool; returns the status (OK, QUOTA_EXCEEDED, INVALID_INPUT)."""
        return int(self._lib.fj_kvpool_fork(self._h, src_lane, src_logical_len, dst_lane, prefix_tokens, reserved_tokens))

    def cow_tail(self, lane: int, logical_len: int):
        """PagedSequence::cow_tail; returns (status, copied, source page, destination page, rows to copy)."""
        out = (C.c_uint32 * 4)()
        status = int(self._lib.fj_kvpool_cow_tail(self._h, lane, logical_len, out))
        return status, bool(out[0]), int(out[1]), int(out[2]), int(out[3])

    def rewind_private(self, lane: int, current_len: int, new_len: int) -> int:
        """PagedSequence::rewind_private as a check: OK, POOL_INVALID_CHECKPOINT or POOL_SHARED_TAIL (the length itself lives with the caller)."""
        return self._lib.fj_kvpool_rewind_private(self._h, lane, current_len, new_len)

    def checkpoint(self, lane: int, logical_len: int) -> "_lib.FjKvCheckpoint":
        cp = _lib.FjKvCheckpoint()
        _check(self._lib.fj_kvpool_checkpoint(self._h, lane, logical_len, C.byref(cp)))
        return cp

    def rollback(self, lane: int, checkpoint) -> Tuple[int, int]:
        """Consumes the checkpoint; returns (status, restored logical length)."""
        length = C.c_uint64(0)
        status = self._lib.fj_kvpool_rollback(self._h, lane, C.byref(checkpoint), C.byref(length))
        return status, length.value

    def drop_checkpoint(self, checkpoint) -> int:
        return self._lib.fj_kvpool_checkpoint_drop(self._h, C.byref(checkpoint))

    def tables_tensor(self) -> Tensor:
        return Tensor(self._lib.fj_kvpool_tables_buffer(self._h), Layout.contiguous(U32, (self.lanes, self.table_pages, 2)), self.lanes * self.table_pages * 8)

    def generations_tensor(self) -> Tensor:
        return Tensor(self._lib.fj_kvpool_generations_buffer(self._h), Layout.contiguous(U32, (self.physical_pages,)), self.physical_pages * 4)

    def pack_step(self, starts: Sequence[int], tokens: Sequence[int], read_back: bool = False):
        st, to = np.ascontiguousarray(starts, np.uint32), np.ascontiguousarray(tokens, np.uint32)
        view = _lib.FjPackView()
        _check(self._lib.fj_pack_step(self._h, st.ctypes.data_as(C.c_void_p), to.ctypes.data_as(C.c_void_p), st.size, C.byref(view)))
        if not read_back:
            return view.rows
        out = {"rows": view.rows}
        lanes = st.size

        def rd(buf, n):
            a = np.zeros(max(n, 1), np.uint32)
            if n:
                _check(self._lib.fj_read(self.backend._h, buf, 0, a.ctypes.data_as(C.c_void_p), n * 4))
            return a[:n]
        for name in ("logical_lengths", "query_starts", "absolute_positions", "activity"):
            out[name] = rd(getattr(view, name), lanes)
        out["cu_seqlens"] = rd(view.cu_seqlens, lanes + 1)
        for name in ("positions", "slot_mapping", "row_lane"):
            out[name] = rd(getattr(view, name), view.rows)
        return out


class DenseModel:
    """Dense decoder on the fast path (fj_dense_model_create / fj_dense_step)."""

    def __init__(self, backend: CudaBackend, pool: KvPool, config: dict, embed: Tensor, final_norm: Tensor, layers: Sequence[dict]):
        self.backend, self.pool, self._lib, self.config = backend, pool, backend._lib, dict(config)
        cfg = _lib.FjDenseConfig()
        for key in ("dtype", "layers", "hidden", "q_heads", "kv_heads", "head_dim", "intermediate", "vocab", "qk_norm", "eps", "theta", "max_rows"):
            setattr(cfg, key, config[key])
        arr = (_lib.FjDenseLayerWeights * len(layers))()
        for i, layer in enumerate(layers):
            for name, _ in _lib.FjDenseLayerWeights._fields_:
                setattr(arr[i], name, layer[name].buffer if layer.get(name) is not None else 0)
        handle = C.c_void_p()
        _check(self._lib.fj_dense_model_create(backend._h, C.byref(cfg), embed.buffer, final_norm.buffer, arr, pool._h, C.byref(handle)))
        self._h = handle

    def close(self):
        if getattr(self, "_h", None) and getattr(self.backend, "_h", None):
            self._lib.fj_dense_model_destroy(self._h)
        self._h = None

    def step(self, token_ids=None, want_tokens: bool = True, logits: Optional[Tensor] = None, lanes: Optional[int] = None):
        ids = None if token_ids is None else np.ascontiguousarray(token_ids, np.uint32)
        out = np.zeros(lanes if lanes is not None else self.pool.lanes, np.uint32) if want_tokens else None
        _check(self._lib.fj_dense_step(self._h, None if ids is None else ids.ctypes.data_as(C.c_void_p),
                                       None if out is None else out.ctypes.data_as(C.c_void_p), logits.buffer if logits is not None else 0))
        return out

    def fill_kv(self, seed: int = 0):
        _check(self._lib.fj_dense_fill_kv(self._h, seed))

    def graph_replay(self, enabled: bool = True):
        """Decode-only steps are recorded once per launch-geometry bucket as a CUDA graph and replayed (fj_dense_graph_replay)."""
        _check(self._lib.fj_dense_graph_replay(self._h, int(enabled)))

    def graph_stats(self):
        a, b, c = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
        _check(self._lib.fj_dense_graph_stats(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return {"recordings": a.value, "replays": b.value, "failures": c.value}

    def kv_pages(self, layer: int, plane: int, first_page: int, count: int, data: Optional[np.ndarray] = None) -> np.ndarray:
        """Reads (data None) or writes the rows of `count` consecutive physical pages of one layer's K (plane 0) or V (plane 1)
        plane; storage values [count, page_tokens, kv_heads * head_dim] (bf16/f16 as uint16 bit patterns)."""
        cfg = self.config
        shape = (count, self.pool.page_tokens, cfg["kv_heads"] * cfg["head_dim"])
        host = np.empty(shape, NP_OF[cfg["dtype"]]) if data is None else np.ascontiguousarray(data, NP_OF[cfg["dtype"]]).reshape(shape)
        _check(self._lib.fj_dense_kv_pages(self._h, layer, plane, first_page, count, host.ctypes.data_as(C.c_void_p), 0 if data is None else 1))
        return host

    def copy_page(self, src_page: int, dst_page: int, tokens: int):
        _check(self._lib.fj_dense_copy_page(self._h, src_page, dst_page, tokens))

    def profile_attention(self, enabled: bool):
        _check(self._lib.fj_dense_profile_attention(self._h, int(enabled)))

    def attention_time(self):
        ns, n = C.c_uint64(0), C.c_uint64(0)
        _check(self._lib.fj_dense_attention_time(self._h, C.byref(ns), C.byref(n)))
        return ns.value, n.value

    def stats(self):
        k, w = C.c_uint64(0), C.c_uint64(0)
        _check(self._lib.fj_dense_step_stats(self._h, C.byref(k), C.byref(w)))
        return {"kernels": k.value, "attn_work_items": w.value}


def nccl_library_path() -> Optional[str]:
    """Path of the NCCL library bundled with PyTorch's wheels, when there is one."""
    try:
        import nvidia.nccl  # type: ignore
        root = os.path.dirname(nvidia.nccl.__file__) if getattr(nvidia.nccl, "__file__", None) else list(nvidia.nccl.__path__)[0]
        path = os.path.join(root, "lib", "libnccl.so.2")
        return path if os.path.exists(path) else None
    except Exception:
        return None


class ExpertParallel:
    """Group of ranks (one per GPU) that share the experts of a sparse-MoE model (fj_ep_*).
    ``exchange`` moves the 128-byte group id from rank 0 to every rank (e.g. a torch.distributed
    broadcast): it receives rank 0's bytes (None elsewhere) and returns the agreed bytes."""

    def __init__(self, backend: CudaBackend, rank: int, world: int, exchange):
        self.backend, self._lib, self.rank, self.world = backend, backend._lib, rank, world
        path = nccl_library_path()
        _check(self._lib.fj_ep_load(path.encode() if path else None))
        mine = None
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            _check(self._lib.fj_ep_unique_id(buf))
            mine = bytes(buf)
        agreed = exchange(mine)
        handle = C.c_void_p()
        _check(self._lib.fj_ep_create(backend._h, (C.c_uint8 * 128).from_buffer_copy(agreed), rank, world, C.byref(handle)))
        self._h = handle

    def all_to_all(self, send: Tensor, recv: Tensor, bytes_per_peer: int):
        _check(self._lib.fj_ep_all_to_all(self._h, send.buffer, recv.buffer, bytes_per_peer))

    def close(self):
        if getattr(self, "_h", None) and getattr(self.backend, "_h", None):
            self._lib.fj_ep_destroy(self._h)
        self._h = None


def _quant_weight(triple) -> "_lib.FjQuantWeight":
    w = _lib.FjQuantWeight()
    w.packed, w.scales, w.biases = (t.buffer for t in triple)
    return w


class MoeModel:
    """Sparse-MoE decoder on the fast path (fj_moe_model_create / fj_moe_step). Quantised weights
    are (packed, scales, biases) tensor triples; ``layers`` entries carry input_norm, q_norm,
    k_norm, post_norm and the triples qkv, o, router, gate, up, down."""

    def __init__(self, backend: CudaBackend, pool: KvPool, config: dict, embed, final_norm: Tensor, lm_head, layers: Sequence[dict],
                 ep: Optional[ExpertParallel] = None):
        self.backend, self.pool, self._lib, self.config = backend, pool, backend._lib, dict(config)
        cfg = _lib.FjMoeConfig()
        for name, _ in _lib.FjMoeConfig._fields_:
            setattr(cfg, name, config.get(name, 0))
        arr = (_lib.FjMoeLayerWeights * len(layers))()
        for i, layer in enumerate(layers):
            for name in ("input_norm", "q_norm", "k_norm", "post_norm"):
                setattr(arr[i], name, layer[name].buffer)
            for name in ("qkv", "o", "router", "gate", "up", "down"):
                setattr(arr[i], name, _quant_weight(layer[name]))
        e, h = _quant_weight(embed), _quant_weight(lm_head)
        handle = C.c_void_p()
        _check(self._lib.fj_moe_model_create(backend._h, C.byref(cfg), C.byref(e), final_norm.buffer, C.byref(h), arr, pool._h, ep._h if ep is not None else None,
                                             C.byref(handle)))
        self._h = handle

    def connect_peers(self, all_gather) -> bool:
        """Switches an expert-parallel model to the direct exchange (peer stores over NVLink instead of NCCL, no host
        round trip; fj_moe_ep_*). ``all_gather(obj) -> list`` returns every rank's object in rank order (e.g.
        torch.distributed.all_gather_object); it is called three times here and once more by close(). Returns whether
        the direct exchange is in use: every rank must have mapped every peer, otherwise all stay on NCCL."""
        mine = (C.c_uint8 * 320)()
        status = self._lib.fj_moe_ep_export(self._h, mine)
        table = all_gather(bytes(mine) if status == 0 else None)
        if status == 0 and all(t is not None and len(t) == 320 for t in table):
            status = self._lib.fj_moe_ep_connect(self._h, (C.c_uint8 * (320 * len(table))).from_buffer_copy(b"".join(table)))
        else:
            status = status or 1
        self._peer_gather = all_gather
        everyone = all(s == 0 for s in all_gather(int(status)))
        if everyone:
            _check(self._lib.fj_moe_ep_direct(self._h, 1))
        all_gather(None)  # nobody steps before everybody has switched
        return everyone

    def set_wait_polls(self, polls: int):
        _check(self._lib.fj_moe_ep_wait_polls(self._h, polls))

    def uniform_routing(self, enabled: bool):
        """Measurement aid: replace the router's choice by an even spread over the experts (fj_moe_uniform_routing)."""
        _check(self._lib.fj_moe_uniform_routing(self._h, int(enabled)))

    def received_rows(self) -> np.ndarray:
        """Direct exchange: rows this rank received for its experts in the last step, [layers, chunks]."""
        chunks = max(1, int(self.config.get("ep_chunks", 0) or 1))
        out = np.zeros(self.config["layers"] * chunks, np.uint32)
        _check(self._lib.fj_moe_ep_received(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out.reshape(self.config["layers"], chunks)

    def set_return_mode(self, mode: int):
        """Direct exchange: 0 or 1 = the origin reads the results from the owner (default), 2 = the owner writes them."""
        _check(self._lib.fj_moe_ep_return_mode(self._h, mode))

    def close(self):
        if getattr(self, "_h", None) and getattr(self.backend, "_h", None):
            gather = getattr(self, "_peer_gather", None)
            if gather is not None:
                # mappings of the peers' buffers are closed everywhere before anyone frees
                self._lib.fj_moe_ep_disconnect(self._h)
                gather(None)
                self._peer_gather = None
            self._lib.fj_moe_model_destroy(self._h)
        self._h = None

    def step(self, token_ids=None, want_tokens: bool = True, logits: Optional[Tensor] = None, lanes: Optional[int] = None):
        ids = None if token_ids is None else np.ascontiguousarray(token_ids, np.uint32)
        out = np.zeros(lanes if lanes is not None else self.pool.lanes, np.uint32) if want_tokens else None
        _check(self._lib.fj_moe_step(self._h, None if ids is None else ids.ctypes.data_as(C.c_void_p),
                                     None if out is None else out.ctypes.data_as(C.c_void_p), logits.buffer if logits is not None else 0))
        return out

    def capture_routes(self, enabled: bool = True):
        _check(self._lib.fj_moe_capture_routes(self._h, int(enabled)))

    def routes(self, layer: int, rows: int):
        """(expert ids u32 [rows, top_k], weights f32 [rows, top_k]) of one layer of the last step."""
        k = self.config["top_k"]
        experts, weights = np.zeros((rows, k), np.uint32), np.zeros((rows, k), np.float32)
        _check(self._lib.fj_moe_read_routes(self._h, layer, rows, experts.ctypes.data_as(C.c_void_p), weights.ctypes.data_as(C.c_void_p)))
        return experts, weights

    def stats(self):
        k, w = C.c_uint64(0), C.c_uint64(0)
        _check(self._lib.fj_moe_step_stats(self._h, C.byref(k), C.byref(w)))
        return {"kernels": k.value, "attn_work_items": w.value}

    def phase_timing(self, enabled: bool):
        _check(self._lib.fj_moe_phase_timing(self._h, 1 if enabled else 0))

    def phase_ms(self):
        """Milliseconds of the last step summed over the layers: attention + router, dispatch, experts, return + combine."""
        out = (C.c_float * 4)()
        _check(self._lib.fj_moe_read_phase_ms(self._h, out))
        return [float(v) for v in out]
