"""Layout, aliasing and scalar rules shared by the ops (the contract of the reference's
src/zig_cu_kernels/torch/common.py: exact aliases are legal, other overlap goes through a temporary, outputs that
share memory are errors, Python scalars round once to FP32), plus the split-K workspace cache."""

import math
import threading

import torch

GROUP = 128
ALIGN = 16
SCALE_DTYPES = (torch.float32, torch.float8_e8m0fnu)
KINDS = {torch.bfloat16: 0, torch.float32: 1, torch.float8_e4m3fn: 2}
FP32_LIMIT = 2**128 - 2**103  # least magnitude that rounds to infinity in FP32


def raw_stream(device_index):
    """The `cudaStream_t` of PyTorch's current stream on `device_index`, without building a Stream object."""
    return torch._C._cuda_getCurrentRawStream(device_index)


# ---- argument checks -------------------------------------------------------------------------------------------

def need_tensor(name, value):
    if not isinstance(value, torch.Tensor):
        raise TypeError(f"{name} must be a tensor, got {type(value).__name__}")


def need_dtype(name, tensor, allowed):
    if tensor is not None and tensor.dtype not in allowed:
        raise ValueError(f"{name} must be a {' or '.join(str(d) for d in allowed)} tensor, got {tensor.dtype}")


def need_choice(name, value, allowed):
    if value not in allowed:
        raise ValueError(f"{name} must be one of {', '.join(str(a) for a in allowed)}, got {value}")


def need_below(limit, **sizes):
    for name, size in sizes.items():
        if size >= limit:
            raise ValueError(f"{name} = {size} must be below {limit}")


def common_cuda_device(named):
    """Device index shared by the tensors of `named` ((name, tensor) pairs, None skipped); ValueError otherwise."""
    first_name, first = named[0]
    if not first.is_cuda:
        raise ValueError(f"{first_name} must be a CUDA tensor, got a tensor on {first.device}")
    index = first.get_device()
    for name, tensor in named[1:]:
        if tensor is not None and (not tensor.is_cuda or tensor.get_device() != index):
            raise ValueError(f"{name} must be on cuda:{index}, the device of {first_name}, got {tensor.device}")
    return index


def same_device(named):
    """Fake-mode twin of `common_cuda_device`: compares `.device` only."""
    first_name, first = named[0]
    for name, tensor in named[1:]:
        if tensor is not None and tensor.device != first.device:
            raise ValueError(f"{name} must be on {first.device}, the device of {first_name}, got {tensor.device}")


def _int_to_fp32(value):
    """Nearest-even FP32 value of a Python int, without passing through a double."""
    magnitude = abs(value)
    extra = magnitude.bit_length() - 24
    if extra <= 0:
        return float(value)
    head, tail = divmod(magnitude, 1 << extra)
    half = 1 << (extra - 1)
    if tail > half or (tail == half and head % 2 == 1):
        head += 1
    return math.copysign(float(head << extra), value)


def fp32_scalar(name, value):
    """`value` as a Python float that converts to the FP32 value nearest to `value`. TypeError for anything but a
    Python int or float; OverflowError when a finite value rounds to infinity."""
    if isinstance(value, (torch.SymFloat, torch.SymInt)):
        return value
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise TypeError(f"{name} must be a Python number, got {type(value).__name__}")
    if isinstance(value, float):
        if math.isfinite(value) and abs(value) >= FP32_LIMIT:
            raise OverflowError(f"{name} = {value} rounds to infinity in FP32")
        return value
    if abs(value) >= FP32_LIMIT:
        raise OverflowError(f"{name} = {value} rounds to infinity in FP32")
    return _int_to_fp32(value)


def python_int(name, value):
    if isinstance(value, torch.SymInt) or type(value) is int:
        return value
    raise TypeError(f"{name} must be a Python int, got {type(value).__name__}")


# ---- layouts ---------------------------------------------------------------------------------------------------

def rows_of_leading(tensor):
    """(row count, row stride in elements) when the leading dimensions flatten into rows of one stride, else None.
    One row or none has stride 0."""
    shape, strides = tensor.shape, tensor.stride()
    if tensor.numel() == 0:
        return math.prod(shape[:-1]), 0
    count, step = 1, 0
    for axis in reversed(range(len(shape) - 1)):
        if shape[axis] == 1:
            continue
        if count == 1:
            step = strides[axis]
        elif strides[axis] != step * count:
            return None
        count *= shape[axis]
    return (count, step) if count > 1 else (count, 0)


def row_matrix(tensor, align=ALIGN):
    """(rows, row stride in elements) when a kernel can address `tensor` in place: last dimension contiguous, one row
    stride, base address and row stride multiples of `align` bytes. None otherwise."""
    if tensor.dim() == 0:
        return None
    width = tensor.shape[-1]
    if width > 1 and tensor.stride(-1) != 1:
        return None
    rows = rows_of_leading(tensor)
    if rows is None or tensor.data_ptr() % align:
        return None
    count, step = rows
    if count > 1 and ((step * tensor.element_size()) % align or step >= 1 << 32):
        return None
    return count, step


def readable_rows(tensor, align=ALIGN):
    """`tensor` or a contiguous copy that `row_matrix` accepts, with its row stride."""
    rows = row_matrix(tensor, align)
    if rows is None:
        tensor = tensor.clone(memory_format=torch.contiguous_format)
        rows = row_matrix(tensor, align)
        if rows is None:  # a 0-d tensor, or an allocation that is not 16-byte aligned: cannot happen for CUDA memory
            raise ValueError("the tensor cannot be laid out as aligned rows")
    return tensor, rows[1]


def writable_rows(tensor, align=ALIGN):
    """Row stride when a kernel may write rows of `tensor` in place (rows must not overlap each other)."""
    rows = row_matrix(tensor, align)
    if rows is None:
        return None
    count, step = rows
    if count > 1 and step < tensor.shape[-1]:
        return None
    return step


def block_scales_like(x, dtype):
    """Empty activation scales `(m, k/128)` with strides `(1, m)`: one column per scale group, rows contiguous."""
    return x.new_empty((x.shape[-1] // GROUP, math.prod(x.shape[:-1])), dtype=dtype).t()


# ---- memory overlap --------------------------------------------------------------------------------------------

def byte_extent(tensor):
    """[start, end) of the bytes `tensor` can touch, or None for an empty tensor."""
    if tensor.numel() == 0:
        return None
    reach = sum((size - 1) * stride for size, stride in zip(tensor.shape, tensor.stride()) if stride > 0)
    low = sum((size - 1) * stride for size, stride in zip(tensor.shape, tensor.stride()) if stride < 0)
    start = tensor.data_ptr() + low * tensor.element_size()
    return start, tensor.data_ptr() + (reach + 1) * tensor.element_size()


def extents_overlap(first, second):
    a, b = byte_extent(first), byte_extent(second)
    return a is not None and b is not None and a[0] < b[1] and b[0] < a[1]


def same_view(first, second):
    return (first.data_ptr() == second.data_ptr() and first.dtype == second.dtype and first.shape == second.shape
            and first.stride() == second.stride())


def writes_in_place(output, inputs, aliases=()):
    """True when a kernel may write `output` while it reads `inputs` and `aliases`: no overlap with an input, and
    overlap with an alias only as the very same view."""
    for tensor in inputs:
        if tensor is not None and extents_overlap(output, tensor):
            return False
    for tensor in aliases:
        if tensor is not None and extents_overlap(output, tensor) and not same_view(output, tensor):
            return False
    return True


def _row_form(tensor):
    """(rows, row bytes, row stride in bytes) for tensors of contiguous rows of one stride; None otherwise."""
    size = tensor.element_size()
    if tensor.dim() == 0:
        return 1, size, 0
    if tensor.shape[-1] > 1 and tensor.stride(-1) != 1:
        return None
    rows = rows_of_leading(tensor)
    if rows is None:
        return None
    return rows[0], tensor.shape[-1] * size, rows[1] * size


def share_memory(first, second):
    """Whether some byte belongs to an element of both tensors. Exact for two row-form tensors with equal row strides
    (or one single row); otherwise the answer of the byte extents."""
    if not extents_overlap(first, second):
        return False
    a, b = _row_form(first), _row_form(second)
    if a is None or b is None:
        return True
    (rows_a, width_a, step_a), (rows_b, width_b, step_b) = a, b
    if rows_a > 1 and rows_b > 1 and step_a != step_b:
        return True
    step = step_a if rows_a > 1 else step_b
    if step <= 0:
        return True
    # row i of `first` covers [i*step, i*step + width_a); row j of `second` covers [delta + j*step, ... + width_b).
    # They intersect when -width_b < delta + (j - i) * step < width_a for some i, j in range, d = j - i.
    delta = second.data_ptr() - first.data_ptr()
    d_low = (-width_b - delta) // step + 1
    d_high = -((delta - width_a) // step) - 1
    return max(d_low, 1 - rows_a) <= min(d_high, rows_b - 1)


def overlaps_itself(tensor):
    """Whether two elements of `tensor` share memory (exact when, sorted by stride, each stride clears the span of the
    smaller ones, or for two non-trivial dimensions; True otherwise)."""
    if tensor.is_contiguous():
        return False
    dims = sorted((stride, size) for size, stride in zip(tensor.shape, tensor.stride()) if size > 1)
    span = 0
    for stride, size in dims:
        if stride <= span:
            break
        span += (size - 1) * stride
    else:
        return False
    if len(dims) != 2 or dims[0][0] == 0:
        return True
    (s0, n0), (s1, n1) = dims
    g = math.gcd(s0, s1)
    return s1 // g < n0 and s0 // g < n1


def need_separate_outputs(names, outputs):
    for i, output in enumerate(outputs):
        if output is None:
            continue
        if overlaps_itself(output):
            raise ValueError(f"the elements of {names[i]} share memory")
        for j in range(i + 1, len(outputs)):
            if outputs[j] is not None and share_memory(output, outputs[j]):
                raise ValueError(f"{names[i]} and {names[j]} share memory")


# ---- split-K workspace -----------------------------------------------------------------------------------------

class Workspace:
    """FP32 partial tiles and zeroed tile counters of one (device, stream). A thread holds it in a `with` block until
    every launch that uses the addresses is queued. The kernels leave the counters at zero."""

    def __init__(self, device_index, private_pools):
        self.device_index = device_index
        self.private_pools = private_pools
        self.lock = threading.Lock()
        self.holder = None
        self.pools = []
        self.parts = torch.empty(0, dtype=torch.uint8, device=device_index)
        self.counters = torch.zeros(0, dtype=torch.int32, device=device_index)

    def __enter__(self):
        self.lock.acquire()
        self.holder = threading.get_ident()
        return self

    def __exit__(self, *exc):
        self.holder = None
        self.lock.release()

    def addresses(self, part_bytes, counter_count):
        if self.holder != threading.get_ident():
            raise RuntimeError("a thread must hold the workspace while it uses the addresses")
        if self.parts.numel() < part_bytes or self.counters.numel() < counter_count:
            if self.private_pools:
                # A pool of its own keeps the buffers out of whatever pool PyTorch routes this thread to (for
                # example the pool of a CUDA-graph tree of torch.compile).
                with torch.cuda.device(self.device_index):
                    pool = torch.cuda.MemPool()
                self.pools.append(pool)
                with torch.cuda.use_mem_pool(pool, self.device_index):
                    self._grow(part_bytes, counter_count)
            else:
                self._grow(part_bytes, counter_count)
        return self.parts.data_ptr(), self.counters.data_ptr()

    def _grow(self, part_bytes, counter_count):
        if self.parts.numel() < part_bytes:
            self.parts = torch.empty(max(part_bytes, 2 * self.parts.numel()), dtype=torch.uint8,
                                     device=self.device_index)
        if self.counters.numel() < counter_count:
            self.counters = torch.zeros(max(counter_count, 2 * self.counters.numel()), dtype=torch.int32,
                                        device=self.device_index)


MAX_EAGER_WORKSPACES = 16
_eager = {}
_eager_lock = threading.Lock()


def workspace_for(device_index, stream):
    """Workspace of a call on `stream`: a fresh one inside a CUDA graph capture (it lives in the graph's pool), else
    the cached one of this (device, stream)."""
    if torch.cuda.is_current_stream_capturing():
        return Workspace(device_index, private_pools=False)
    key = (device_index, stream)
    with _eager_lock:
        workspace = _eager.get(key)
        if workspace is None:
            if len(_eager) >= MAX_EAGER_WORKSPACES:
                _eager.pop(next(iter(_eager)))
            workspace = _eager[key] = Workspace(device_index, private_pools=True)
        return workspace
