"""Helpers shared by the GPU parity tests."""
import torch

from oracle import dge_oracle as O


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| / max |b| in float64."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def load_block(blk, weights, device, dtype):
    blk.load_state_dict(weights, strict=True)
    blk.eval()
    return blk.to(device=device, dtype=dtype)


def strip_col2_of_extra(p: torch.Tensor) -> torch.Tensor:
    """Column 2 of extra-token rows is unwritten in the reference; zero it for comparison."""
    p = p.clone()
    p[p[:, 1] < 0, 2] = 0
    return p


def random_indices(B, Hr, Wr, n_splits, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, n_splits, (B, Hr, Wr), generator=g)


__all__ = ["O", "rel_err", "load_block", "strip_col2_of_extra", "random_indices"]
