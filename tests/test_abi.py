"""CPU checks of the C-ABI boundary: the library builds and loads, exports every symbol
the header declares, and rejects bad arguments on the host with the documented codes
(no kernel is launched)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from vtpack_b200 import build
    build.build()
    from vtpack_b200 import _lib
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "vtpack_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vtp_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert getattr(lib, n) is not None


def test_bindings_cover_header(lib):
    from vtpack_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == _declared()


def test_version_and_error_string(lib):
    assert lib.vtp_version() >= 1000
    assert isinstance(lib.vtp_last_error_string(), bytes)


def test_null_and_shape_errors(lib):
    from vtpack_b200 import _lib
    # null pointers
    assert lib.vtp_router_gate(None, 0, 1, 16, 16, 64, 1, 4, None, None, 3, None, None, None) == -1
    assert b"null" in lib.vtp_last_error_string()
    assert lib.vtp_pool(None, 0, 1, 257, 64, 16, 1, None, None, 10, None, None, None, 0.0, None, None, None) == -1
    assert lib.vtp_linear(None, 8, None, None, None, 0, None, 8, 0, 4, None, 8, 8, 0, None) == -1
    # bad dtype / shape, with fake but aligned non-null pointers (never dereferenced on the host)
    p = ctypes.c_void_p(4096)
    assert lib.vtp_router_gate(p, 7, 1, 16, 16, 64, 1, 4, p, p, 3, None, p, None) == -3
    assert lib.vtp_router_gate(p, 0, 1, 15, 16, 64, 1, 4, p, p, 3, None, p, None) == -2
    assert lib.vtp_layernorm(p, 1, 4, None, 60, 60, p, p, 1e-6, p, None) == -2      # C not 16-byte multiple
    q = ctypes.c_void_p(4100)
    assert lib.vtp_layernorm(q, 1, 4, None, 64, 64, p, p, 1e-6, p, None) == -4      # unaligned
    splits = (ctypes.c_int * 3)(4, 3, 1)
    assert lib.vtp_index_to_patch(p, 0, splits, 3, 1, 4, 4, 4, 1, p, p, p, None, None) == -2  # 3 does not divide 4
    s = _lib.DgeShape()
    assert lib.vtp_block_workspace_bytes(ctypes.byref(s)) == -1
    # a stage of blocks in one call: null arrays, no blocks, a workspace that is too small
    s.dtype, s.B, s.H, s.W, s.num_extra, s.C, s.heads, s.hidden, s.region, s.n_splits = 1, 4, 16, 16, 0, 64, 1, 512, 4, 3
    s.splits[0], s.splits[1], s.splits[2] = 4, 2, 1
    w = (_lib.BlockWeights * 2)()
    assert lib.vtp_dge_blocks_forward(ctypes.byref(s), None, 2, p, p, None, p, 1 << 30, None) == -1
    assert lib.vtp_dge_blocks_forward(ctypes.byref(s), w, 0, p, p, None, p, 1 << 30, None) == -2
    assert lib.vtp_dge_blocks_forward(ctypes.byref(s), w, 2, p, p, None, p, 16, None) == -2
    assert b"workspace" in lib.vtp_last_error_string()


def test_workspace_size_formula(lib):
    from vtpack_b200 import _lib
    s = _lib.DgeShape()
    s.dtype, s.B, s.H, s.W, s.num_extra, s.C, s.heads, s.hidden, s.region, s.n_splits = 1, 4, 16, 16, 1, 192, 3, 768, 4, 3
    s.splits[0], s.splits[1], s.splits[2] = 4, 2, 1
    n = lib.vtp_block_workspace_bytes(ctypes.byref(s))
    rows = 4 * 257
    lower = rows * 2 * (192 * 6 + 2 * 192 + 768)
    assert lower <= n <= lower + rows * (16 * 8 + 32) + 64 * 1024   # + row statistics (16 slot pairs) and index lists


def test_missing_library_fails_loudly(monkeypatch):
    from vtpack_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libvtpack_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_cpu_tensors_rejected():
    import torch
    from vtpack_b200.layers import grained_sample_compress
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        grained_sample_compress(torch.zeros(1, 17, 8), torch.zeros(2, 4, dtype=torch.int64), 4, 4, 1)


def test_complexity_accounting_matches_reference_fixture():
    """VisionTransformer.complexity() of the mirror, fed the per-image query counts of the golden
    forward the way the fused kernels leave them, reproduces the MACs the reference's own
    complexity() reported for that forward (deit_dge.py:233-249, dge.py:40-59)."""
    import os
    import numpy as np
    import torch
    from vtpack_b200.models.dge.deit_dge import deit_dge_s124_tiny_patch16_256
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "model_tiny_fp32.npz"))
    m = deit_dge_s124_tiny_patch16_256().eval()
    counts = torch.from_numpy(g["batch_lengths"]).int()
    tokens = torch.empty(0).expand(2, 257, 0)
    for i, blk in enumerate(m.blocks):
        blk.dge.states.update({"batches_device": counts[i], "input": tokens, "gate": None, "size": (16, 16),
                               "num_extra_tokens": 1})
    comp = m.complexity(torch.empty(2, 3, 256, 256))
    assert float(comp["static"]) == float(g["comp_static"])
    assert float(comp["dynamic"]) == float(g["comp_dynamic"])
