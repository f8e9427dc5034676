"""Seeded synthetic weights and inputs for benchmarks and smoke runs.

ImageNet and the trained checkpoints of the reference are not available offline, so
throughput is measured on random-init models of the same architecture and N(0,1)
images of the same shape: every weight matrix, the cls token and the position
embedding trunc-normal(std 0.02), LayerNorm weights 1, all biases (the gate's too) 0.
"""
from typing import Dict, Sequence

import torch

ARCH = {
    "tiny": dict(embed_dim=192, depth=12, num_heads=3),
    "small": dict(embed_dim=384, depth=12, num_heads=6),
    "base": dict(embed_dim=768, depth=12, num_heads=12),
}


def state_dict(embed_dim: int, depth: int, num_heads: int, img_size: int = 256, patch: int = 16,
               num_classes: int = 1000, mlp_ratio: int = 4, split_sizes: Sequence[int] = (4, 2, 1),
               seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)

    def tn(*shape):
        t = torch.empty(*shape)
        torch.nn.init.trunc_normal_(t, std=std, a=-2 * std, b=2 * std, generator=g)
        return t

    C = embed_dim
    sd = {"cls_token": tn(1, 1, C), "pos_embed": tn(1, (img_size // patch) ** 2 + 1, C),
          "patch_embed.proj.weight": tn(C, 3, patch, patch), "patch_embed.proj.bias": torch.zeros(C)}
    for i in range(depth):
        p = f"blocks.{i}."
        sd.update({
            p + "norm1.weight": torch.ones(C), p + "norm1.bias": torch.zeros(C),
            p + "attn.q.weight": tn(C, C), p + "attn.q.bias": torch.zeros(C),
            p + "attn.kv.weight": tn(2 * C, C), p + "attn.kv.bias": torch.zeros(2 * C),
            p + "attn.proj.weight": tn(C, C), p + "attn.proj.bias": torch.zeros(C),
            p + "norm2.weight": torch.ones(C), p + "norm2.bias": torch.zeros(C),
            p + "mlp.fc1.weight": tn(mlp_ratio * C, C), p + "mlp.fc1.bias": torch.zeros(mlp_ratio * C),
            p + "mlp.fc2.weight": tn(C, mlp_ratio * C), p + "mlp.fc2.bias": torch.zeros(C),
            p + "dge.splits": torch.tensor(list(split_sizes)),
            p + "dge.router.gate.weight": tn(len(split_sizes), C),
            p + "dge.router.gate.bias": torch.zeros(len(split_sizes)),
        })
    sd.update({"norm.weight": torch.ones(C), "norm.bias": torch.zeros(C),
               "head.weight": tn(num_classes, C), "head.bias": torch.zeros(num_classes)})
    return sd


def images(batch: int, img_size: int = 256, seed: int = 1, pin: bool = False) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, 3, img_size, img_size, generator=g)
    return x.pin_memory() if pin else x


def build_model(kind: str, device, dtype, img_size: int = 256, seed: int = 0, depth=None):
    """A DeiT+DGE (s124) model of the named size with seeded weights, in eval mode."""
    from .models.dge.deit_dge import VisionTransformer
    a = dict(ARCH[kind])
    if depth is not None:
        a["depth"] = depth
    m = VisionTransformer(img_size=img_size, patch_size=16, embed_dim=a["embed_dim"], depth=a["depth"],
                          num_heads=a["num_heads"], mlp_ratio=4, qkv_bias=True, split_sizes=[4, 2, 1])
    m.load_state_dict(state_dict(a["embed_dim"], a["depth"], a["num_heads"], img_size=img_size, seed=seed))
    return m.eval().to(device=device, dtype=dtype)
