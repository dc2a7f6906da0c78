"""Deterministic stand-ins for trained weights, shared by the fixture generator and the tests.

A tensor is a pure function of its name and shape, so a fixture does not have to carry the
weights of a large model: both sides rebuild them.  Scales follow the usual initialisers
(xavier-like for matrices, ones for LayerNorm weights, small noise for biases and embeddings).
"""

import hashlib

import torch


def _canonical(name: str) -> str:
    # the reference registers the routing projections under two names that share one tensor
    # (grm/core/gating_unit.py:35-38); both names must map to the same values
    return name.replace("gating_unit.query_proj.", "gating_unit.query_projection.").replace(
        "gating_unit.key_proj.", "gating_unit.key_projection.")


def seeded_tensor(name: str, shape, device="cpu") -> torch.Tensor:
    name = _canonical(name)
    seed = int.from_bytes(hashlib.sha256(name.encode()).digest()[:4], "little")
    g = torch.Generator().manual_seed(seed)
    shape = tuple(shape)
    if name.endswith("layer_norm.weight"):
        t = 1.0 + 0.1 * torch.randn(shape, generator=g)
    elif len(shape) == 2 and "embedding" not in name:
        bound = (6.0 / (shape[0] + shape[1])) ** 0.5
        t = (torch.rand(shape, generator=g) * 2.0 - 1.0) * bound
    elif "embedding" in name:
        t = torch.randn(shape, generator=g)
    else:
        t = 0.05 * torch.randn(shape, generator=g)
    return t.to(device)


def seeded_state_dict(shapes: dict, device="cpu") -> dict:
    return {name: seeded_tensor(name, shape, device) for name, shape in shapes.items()}


def zipf_token_ids(batch: int, seq_len: int, vocab: int, s: float = 1.1, seed: int = 0) -> torch.Tensor:
    """Token ids with probability proportional to rank^-s (rank 1 = id 0)."""
    g = torch.Generator().manual_seed(seed)
    p = torch.arange(1, vocab + 1, dtype=torch.float64) ** (-s)
    return torch.multinomial(p / p.sum(), batch * seq_len, replacement=True, generator=g).view(batch, seq_len)
