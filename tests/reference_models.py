"""Builders shared by the drop-in test and its CPU arm: the reference's own model classes, seeded.

``build(name)`` returns ``(model, x)`` on the CPU: the single-layer adding-problem model of
configuration 1 (``SegmentRecurrentMemoryModel``, B=2, T=512, segment 128, hidden 128, key dim 64,
top-k 2) or a two-layer ``HierarchicalSegmentMemoryModel`` (hidden 64, key dim 32, segment 64, top-k 2),
both with fp32 archive storage, no selective recomputation and no dropout.  ``run(model, x)`` does one
forward and one backward pass of ``outputs^2.mean() + memory^2.mean()`` and returns outputs, final
states and every gradient as numpy arrays.

Run as a script it is the CPU arm: it imports the reference package from the folder given with
``--python-path`` -- untouched, so the reference's own PyTorch fallback computes -- and writes the
results of both models to ``--out`` (an ``.npz``).
"""

from __future__ import annotations

import argparse
import sys

import numpy as np
import torch


def adding_problem_inputs(batch, seq_len, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.zeros(batch, seq_len, 2)
    x[:, :, 0] = torch.rand(batch, seq_len, generator=g)
    half = seq_len // 2
    x[torch.arange(batch), torch.randint(0, half, (batch,), generator=g), 1] = 1.0
    x[torch.arange(batch), torch.randint(half, seq_len, (batch,), generator=g), 1] = 1.0
    return x


def build(name):
    import grm

    if name == "single":
        torch.manual_seed(0)
        model = grm.SegmentRecurrentMemoryModel(
            input_size=2, hidden_size=128, output_size=1, segment_length=128, memory_key_dim=64, retrieval_top_k=2,
            memory_capacity_segments=8, memory_storage_dtype=torch.float32, recomputation_ratio=0.0, dropout=0.0)
        return model, adding_problem_inputs(2, 512, seed=0)
    if name == "stack":
        torch.manual_seed(1)
        model = grm.HierarchicalSegmentMemoryModel(
            input_size=64, hidden_size=64, output_size=8, num_layers=2, segment_length=64, memory_key_dim=32,
            retrieval_top_k=2, memory_capacity_segments=8, memory_storage_dtype=torch.float32, recomputation_ratio=0.0,
            dropout=0.0)
        return model, torch.randn(3, 256, 64, generator=torch.Generator().manual_seed(2))
    raise ValueError(name)


def run(model, x):
    model.train()                    # dropout is 0; training mode keeps the autograd path the trainer uses
    x = x.clone().requires_grad_(True)
    outputs, h_final, memory_final, _ = model(x, reset_memory=True)
    loss = outputs.pow(2).mean() + memory_final.pow(2).mean()
    loss.backward()
    result = {"outputs": outputs, "h_final": h_final, "memory_final": memory_final, "loss": loss, "grad::x": x.grad}
    for pname, p in model.named_parameters():
        if p.grad is not None:
            result[f"grad::{pname}"] = p.grad
    return {k: v.detach().float().cpu().numpy() for k, v in result.items()}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--python-path", required=True, help="folder that holds the reference package `grm`")
    parser.add_argument("--out", required=True)
    args = parser.parse_args(argv)
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.python_path)
    torch.set_num_threads(4)
    payload = {}
    for name in ("single", "stack"):
        model, x = build(name)
        for key, value in run(model, x).items():
            payload[f"{name}::{key}"] = value
    np.savez(args.out, **payload)
    return 0


if __name__ == "__main__":
    sys.exit(main())
