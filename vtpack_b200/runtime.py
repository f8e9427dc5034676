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


_scratch = {}       # (device type, index) -> buffer
_scratch_gen = {}   # (device type, index) -> how many times the buffer was replaced
_scratch_users = {}  # (device type, index) -> streams that have been handed the current buffer


def scratch(device, nbytes: int) -> torch.Tensor:
    """A uint8 buffer of at least nbytes on `device`, grown on demand and reused.

    One buffer per device, shared by every block / model forward on it: forwards that can run at
    the same time (two streams, two host threads) would overwrite each other's intermediates, so
    run the forwards of one device on one stream at a time.  When the buffer has to grow, the old
    one is handed back to the allocator only after the streams it was given to have finished
    their queued work; CUDA graphs captured against it are invalid from then on
    (``scratch_generation`` changes)."""
    key = (device.type, device.index)
    buf = _scratch.get(key)
    cur = torch.cuda.current_stream(device)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            for st in _scratch_users.get(key, ()):
                buf.record_stream(st)          # kernels queued on st may still be using the old buffer
        buf = torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)
        _scratch[key] = buf
        _scratch_gen[key] = _scratch_gen.get(key, 0) + 1
        _scratch_users[key] = []
    users = _scratch_users.setdefault(key, [])
    if all(u.cuda_stream != cur.cuda_stream for u in users):
        users.append(cur)
    return buf


def scratch_generation(device) -> int:
    """Changes whenever the device's scratch buffer is replaced by a larger one."""
    return _scratch_gen.get((device.type, device.index), 0)
