"""Device-side plumbing shared by the op wrappers: dtype codes, the current CUDA
stream as a raw pointer, and a cached scratch buffer (PyTorch owns all device memory;
the library never allocates)."""
import torch

from . import _lib


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return _lib.VTP_F32
    if t == torch.bfloat16:
        return _lib.VTP_BF16
    raise TypeError(f"vtpack_b200 supports float32 and bfloat16, got {t}")


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("vtpack_b200 ops run on CUDA tensors only (there is no CPU path)")


def ptr(t):
    return None if t is None else t.data_ptr()


_scratch = {}


def scratch(device, nbytes: int) -> torch.Tensor:
    """A uint8 buffer of at least nbytes on `device`, grown on demand and reused."""
    key = (device.type, device.index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf
