from .deit_dge import (  # noqa: F401
    Attention, Block, Mlp, PatchEmbed, VisionTransformer,
    deit_dge_s124_base_patch16_256, deit_dge_s124_small_patch16_256, deit_dge_s124_tiny_patch16_256,
)
