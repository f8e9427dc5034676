"""Load the reference's own Python modules on a CPU-only machine.

TEST INFRASTRUCTURE ONLY (used when generating golden fixtures and by the
CPU tests that pin the oracle); never imported by the shipped package.

The reference's native extension ``vtpack._C`` is CUDA-only and ``timm`` is
not installed, so two stand-ins are placed in ``sys.modules`` before the
reference is imported from its checkout:

  * ``vtpack._C``: the four functions the eval path calls and the ragged product of the
    training path (``vtpack/layers/csrc/vision.cpp:9-29``), backed by ``oracle/dge_oracle.py``, and the
    four bilinear-attention functions, backed by ``oracle/bilinear_oracle.py``;
  * ``timm.models.{layers,registry,vision_transformer}``: the handful of names
    ``vtpack/models/dge/deit_dge.py:9-11`` imports.  ``PatchEmbed`` is the
    conv(kernel = stride = patch) + flatten + transpose the reference's own
    ``pvt_dge.py:149-179`` also spells out; weight initialisation is a no-op
    because callers load a seeded state_dict afterwards.

The reference's ``dge.py``, ``grained_sample.py``, ``sparse_ops.py``,
``deit_dge.py`` and ``standard/deit.py`` then run unmodified, in eval mode and (with
stochastic depth off) in training mode, backward passes included: the reference's autograd
functions call the same stand-ins.
"""
import importlib
import os
import sys
import types

import torch
from torch import nn

from . import bilinear_oracle, dge_oracle

# a checkout of the reference: $VTPACK_REFERENCE_ROOT, else a directory "reference" beside this repository
REFERENCE_ROOT = os.environ.get("VTPACK_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "vtpack", "layers", "dge.py"))


class _PatchEmbed(nn.Module):
    def __init__(self, img_size=224, patch_size=16, in_chans=3, embed_dim=768):
        super().__init__()
        self.num_patches = (img_size // patch_size) ** 2
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


class _DropPath(nn.Module):
    def __init__(self, p=0.0):
        super().__init__()
        self.p = p

    def forward(self, x):
        assert not self.training or self.p == 0.0, "stand-in has no stochastic depth"
        return x


def _not_on_eval_path(*a, **k):
    raise NotImplementedError("not on the eval path; no CPU stand-in")


def install():
    """Put the stand-ins in sys.modules and the reference checkout on sys.path."""
    if not reference_available():
        raise FileNotFoundError(f"no reference checkout at {REFERENCE_ROOT}")
    if "vtpack._C" in sys.modules:
        return

    timm = types.ModuleType("timm")
    timm_models = types.ModuleType("timm.models")
    layers = types.ModuleType("timm.models.layers")
    layers.PatchEmbed = _PatchEmbed
    layers.DropPath = _DropPath
    layers.trunc_normal_ = torch.nn.init.trunc_normal_
    layers.to_2tuple = lambda v: (v, v) if not isinstance(v, (tuple, list)) else tuple(v)
    registry = types.ModuleType("timm.models.registry")
    registry.register_model = lambda fn: fn
    vit = types.ModuleType("timm.models.vision_transformer")
    vit._cfg = lambda **kw: dict(kw)
    vit._init_vit_weights = lambda *a, **k: None
    timm.models = timm_models
    timm_models.layers = layers
    timm_models.registry = registry
    timm_models.vision_transformer = vit
    for name, mod in (("timm", timm), ("timm.models", timm_models),
                      ("timm.models.layers", layers), ("timm.models.registry", registry),
                      ("timm.models.vision_transformer", vit)):
        sys.modules[name] = mod

    if REFERENCE_ROOT not in sys.path:
        sys.path.insert(0, REFERENCE_ROOT)
    vtpack = importlib.import_module("vtpack")
    c = types.ModuleType("vtpack._C")
    c.grained_sample_index_to_patch = dge_oracle.grained_sample_index_to_patch
    c.grained_sample_compress = dge_oracle.grained_sample_compress
    c.grained_sample_decompress = dge_oracle.grained_sample_decompress
    c.batched_sparse_attention_forward = dge_oracle.batched_sparse_attention_forward
    c.batched_sparse_gemm_forward = dge_oracle.batched_sparse_gemm_forward
    for name in ("bilinear_attention_pointwise_forward", "bilinear_attention_pointwise_backward",
                 "bilinear_attention_channelwise_forward", "bilinear_attention_channelwise_backward"):
        setattr(c, name, getattr(bilinear_oracle, name))
    for name in ("batched_sparse_gemm_v2_forward", "grained_sample_index_to_patch_dense"):
        setattr(c, name, _not_on_eval_path)
    sys.modules["vtpack._C"] = c
    vtpack._C = c


def reference_modules():
    """(layers.dge, layers.grained_sample, models.dge.deit_dge, models.standard.deit)
    of the reference, imported unmodified."""
    install()
    dge = importlib.import_module("vtpack.layers.dge")
    gs = importlib.import_module("vtpack.layers.grained_sample")
    deit_dge = importlib.import_module("vtpack.models.dge.deit_dge")
    deit = importlib.import_module("vtpack.models.standard.deit")
    return dge, gs, deit_dge, deit
