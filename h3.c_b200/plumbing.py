"""PyTorch-side plumbing for one-process-per-GPU hosts: device memory from torch's allocator
wrapped into library tensors, and the two NCCL exchanges of the sequence-parallel /
guidance-group drivers. torch and torch.distributed are passed in by the caller; this module
imports neither, and none of it is needed on a single GPU. No reference counterpart (the
reference is single-device and owns its memory)."""
from __future__ import annotations

from .binding import BF16, F32


class TorchMemory:
    """Device memory from torch (caching allocator), wrapped into library tensors."""

    def __init__(self, torch, gpu, device):
        self.torch, self.gpu, self.device = torch, gpu, device
        self.by_handle = {}

    def bf16(self, elements, fill=None, std=None, generator=None):
        t = self.torch.empty(max(1, elements), dtype=self.torch.bfloat16, device=self.device)
        if std is not None:
            t.normal_(0.0, std, generator=generator)
        elif fill is not None:
            t.fill_(fill)
        else:
            t.zero_()
        wrapped = self.gpu.wrap(t.data_ptr(), elements, BF16)
        self.by_handle[wrapped.handle] = t
        return wrapped

    def f32(self, elements, std=None, generator=None):
        t = self.torch.zeros(max(1, elements), dtype=self.torch.float32, device=self.device)
        if std is not None:
            t.normal_(0.0, std, generator=generator)
        wrapped = self.gpu.wrap(t.data_ptr(), elements, F32)
        self.by_handle[wrapped.handle] = t
        return wrapped

    def torch_of(self, tensor):
        """torch view of a library tensor: the torch allocation it wraps, else a zero-copy byte
        view of the library's own allocation through the CUDA array interface (bytes, because
        the collectives this is used for do not take 16-bit integers)."""
        if tensor.handle not in self.by_handle:
            size = {BF16: 2, F32: 4}[tensor.dtype]

            class _Span:
                __cuda_array_interface__ = {
                    "shape": (tensor.elements * size,), "version": 2, "typestr": "|u1",
                    "data": (tensor.pointer, False)}
            view = self.torch.as_tensor(_Span(), device=self.device)
            self.by_handle[tensor.handle] = view
        return self.by_handle[tensor.handle]

    def release(self, tensor):
        """Drop the torch allocation behind a wrapped tensor (the caller no longer uses it)."""
        self.by_handle.pop(tensor.handle, None)
        tensor.free()


class NcclExchange:
    """all-to-all of equal blocks over NCCL (torch.distributed), on torch's current stream."""

    def __init__(self, dist, memory, world, rank):
        self.dist, self.memory, self.world, self.rank = dist, memory, world, rank
        self.calls = 0

    def all_to_all(self, out, inp):
        self.dist.all_to_all_single(self.memory.torch_of(out), self.memory.torch_of(inp))
        self.calls += 1


class NcclPair:
    """Velocity swap between the two classifier-free-guidance groups: rank i of the cond group
    and rank i of the uncond group exchange their local velocity rows over NCCL."""

    def __init__(self, dist, memory, partner, is_cond):
        self.dist, self.memory, self.partner, self.is_cond = dist, memory, partner, is_cond

    def swap(self, out, inp):
        d = self.dist
        ops = [d.P2POp(d.isend, self.memory.torch_of(inp), self.partner),
               d.P2POp(d.irecv, self.memory.torch_of(out), self.partner)]
        for req in d.batch_isend_irecv(ops):
            req.wait()


def load_bf16_once(dist, memory, gpu, path, file_offset, elements, rank, source=0):
    """Checkpoint tensor for every rank of the node with one pass over the file: the source rank
    reads it from disk into its tensor (the library's chunked, multi-threaded loader), then NCCL
    broadcasts it over NVLink; with N ranks the file system serves 1/N of what N independent
    loads would ask of it (38.5 GB of block weights per rank for the full model). Returns this
    rank's tensor (torch allocation wrapped into a library tensor)."""
    import ctypes as C
    tensor = memory.bf16(elements)
    problem = None
    if rank == source:
        error = C.create_string_buffer(400)
        if not gpu.lib.h3_gpu_tensor_read_file_bf16(tensor.handle, str(path).encode(), file_offset, elements,
                                                    error, len(error)):
            problem = error.value.decode() or "tensor file read failed"
    # every rank learns whether the read worked before anybody enters the collective on garbage
    outcome = [problem]
    dist.broadcast_object_list(outcome, src=source)
    if outcome[0]:
        raise RuntimeError(f"load_bf16_once: {outcome[0]}")
    dist.broadcast(memory.torch_of(tensor), src=source)
    return tensor
