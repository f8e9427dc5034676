"""The allocation-free gate + patch-list entry point (vtp_gate_compact_static).

Collected last on purpose (the file name sorts after every other test file), so a run that
stops at the first failure has already run everything else.

Some callers of the library cannot allocate device memory at all: they are handed their
input and output tensors by a serving framework, or they sit behind an FFI that can carry
device pointers but has no CUDA allocator.  For them the two intermediates of the
gate -> patch-list pipeline live in a fixed array inside the library.  These tests call
the entry point through the C ABI and compare it with the ordinary entry points, which take
the intermediates from the caller.
"""
import ctypes

import pytest
import torch

DEV = "cuda:0"


def _inputs(seed, B=6, G=16, C=384):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, G * G + 1, C, generator=g).bfloat16()
    gw = torch.randn(3, C, generator=g) * 0.05
    gb = torch.randn(3, generator=g) * 0.1
    return x, gw, gb


def _reference_path(lib, _lib, x, gw, gb, B, G, C):
    """vtp_router_gate + vtp_index_to_patch with caller-allocated intermediates."""
    R = (G // 4) ** 2
    idx = torch.empty(B * R, dtype=torch.int32, device=DEV)
    counts = torch.empty(B, dtype=torch.int32, device=DEV)
    offsets = torch.empty(B + 1, dtype=torch.int32, device=DEV)
    patches = torch.zeros(B * (G * G + 1), 4, dtype=torch.int32, device=DEV)
    splits = (ctypes.c_int * 3)(4, 2, 1)
    _lib.check(lib.vtp_router_gate(x.data_ptr(), 1, B, G, G, C, 1, 4, gw.data_ptr(), gb.data_ptr(), 3, None,
                                   idx.data_ptr(), None))
    _lib.check(lib.vtp_index_to_patch(idx.data_ptr(), 0, splits, 3, B, G // 4, G // 4, 4, 1, counts.data_ptr(),
                                      offsets.data_ptr(), patches.data_ptr(), None, None))
    torch.cuda.synchronize()
    return offsets.cpu(), patches.cpu()


@pytest.mark.gpu
def test_static_scratch_matches_caller_scratch_twice():
    from vtpack_b200 import _lib
    lib = _lib.lib()
    B, G, C = 6, 16, 384
    splits = (ctypes.c_int * 3)(4, 2, 1)
    for seed in (21, 22):               # two calls in a row on different inputs: no state may leak
        x, gw, gb = _inputs(seed, B, G, C)
        x, gw, gb = x.to(DEV), gw.to(DEV), gb.to(DEV)
        ref_off, ref_pat = _reference_path(lib, _lib, x, gw, gb, B, G, C)
        offsets = torch.empty(B + 1, dtype=torch.int32, device=DEV)
        patches = torch.zeros(B * (G * G + 1), 4, dtype=torch.int32, device=DEV)
        _lib.check(lib.vtp_gate_compact_static(x.data_ptr(), 1, B, G, G, C, 1, 4, gw.data_ptr(), gb.data_ptr(),
                                               splits, 3, offsets.data_ptr(), patches.data_ptr(), None))
        torch.cuda.synchronize()
        L = int(ref_off[-1])
        assert 17 * B <= L <= 257 * B
        assert torch.equal(offsets.cpu(), ref_off)                 # integer work: bit-exact
        assert torch.equal(patches.cpu()[:L], ref_pat[:L])
        # and against the CPU oracle: the reference's router on the same bf16 tokens, then its patch list
        from oracle import dge_oracle as O
        logits = O.router_forward(x.float().cpu()[:, 1:].reshape(B, G, G, C), gw.cpu(), gb.cpu(), 4)
        top2 = logits.topk(2, -1).values
        assert float((top2[..., 0] - top2[..., 1]).min()) > 1e-5   # no near-tie in these inputs
        o_pat, o_len = O.grained_sample_index_to_patch(logits.argmax(-1), torch.tensor([4, 2, 1]), 4, 1)
        assert torch.equal(offsets.cpu().long()[1:] - offsets.cpu().long()[:-1], o_len)
        assert torch.equal(patches.cpu()[:L].long(), o_pat)


@pytest.mark.gpu
def test_static_scratch_at_its_limits():
    """Exactly 4096 images and 65536 regions (16 x 16 tokens, 4 x 4 regions, 8 channels): both halves of the
    fixed array are used to their last entry, and the result equals the caller-scratch path."""
    from vtpack_b200 import _lib
    lib = _lib.lib()
    B, G, C = 4096, 16, 8
    splits = (ctypes.c_int * 3)(4, 2, 1)
    x, gw, gb = _inputs(23, B, G, C)
    x, gw, gb = x.to(DEV), gw.to(DEV), gb.to(DEV)
    ref_off, ref_pat = _reference_path(lib, _lib, x, gw, gb, B, G, C)
    offsets = torch.empty(B + 1, dtype=torch.int32, device=DEV)
    patches = torch.zeros(B * (G * G + 1), 4, dtype=torch.int32, device=DEV)
    _lib.check(lib.vtp_gate_compact_static(x.data_ptr(), 1, B, G, G, C, 1, 4, gw.data_ptr(), gb.data_ptr(),
                                           splits, 3, offsets.data_ptr(), patches.data_ptr(), None))
    torch.cuda.synchronize()
    L = int(ref_off[-1])
    assert torch.equal(offsets.cpu(), ref_off)
    assert torch.equal(patches.cpu()[:L], ref_pat[:L])


def test_static_scratch_rejects_oversized_calls():
    """Beyond the fixed scratch the call fails on the host with a clear message (no launch)."""
    from vtpack_b200 import _lib
    lib = _lib.lib()
    p = ctypes.c_void_p(4096)
    splits = (ctypes.c_int * 3)(4, 2, 1)
    # 4097 images, and 4096 images x 64 regions: both over the limit
    assert lib.vtp_gate_compact_static(p, 1, 4097, 16, 16, 384, 1, 4, p, p, splits, 3, p, p, None) == -2
    assert b"exceed the static scratch" in lib.vtp_last_error_string()
    assert lib.vtp_gate_compact_static(p, 1, 4096, 32, 32, 384, 1, 4, p, p, splits, 3, p, p, None) == -2
    assert lib.vtp_gate_compact_static(None, 1, 2, 16, 16, 384, 1, 4, p, p, splits, 3, p, p, None) == -1
    # everything the two underlying calls would reject is rejected up front, before the first launch:
    # more than 8192 regions in one image, a split that does not divide the region, an unknown dtype,
    # rows that are not whole 16-byte chunks, an unaligned pointer
    assert lib.vtp_gate_compact_static(p, 1, 1, 512, 512, 384, 1, 4, p, p, splits, 3, p, p, None) == -2
    assert b"8192" in lib.vtp_last_error_string()
    bad_splits = (ctypes.c_int * 3)(4, 3, 1)
    assert lib.vtp_gate_compact_static(p, 1, 2, 16, 16, 384, 1, 4, p, p, bad_splits, 3, p, p, None) == -2
    assert lib.vtp_gate_compact_static(p, 9, 2, 16, 16, 384, 1, 4, p, p, splits, 3, p, p, None) == -3
    assert lib.vtp_gate_compact_static(p, 1, 2, 16, 16, 60, 1, 4, p, p, splits, 3, p, p, None) == -2
    q = ctypes.c_void_p(4100)
    assert lib.vtp_gate_compact_static(q, 1, 2, 16, 16, 384, 1, 4, p, p, splits, 3, p, p, None) == -4
