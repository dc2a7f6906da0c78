"""Generates the golden fixtures in this directory from the reference itself.

Run where a checkout of Sggggt/RNN_with_GRM is available (it is imported, not
copied):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <checkout of Sggggt/RNN_with_GRM>

Every fixture is an ``.npz`` holding seeded inputs and the outputs of the
reference's Python implementation on CPU in float32:

* ``chunk_update_*.npz``  -- ``grm.core.cuda_ops._vectorized_chunk_update`` forward and the
                             autograd gradients of ``h^2.mean() + M^2.mean()`` (the loss of
                             examples/test_grm.py:88).
* ``apply_query.npz``     -- ``_fallback_apply_query`` rank 5 and rank 4 with gradients.
* ``gather.npz``          -- ``_fallback_batched_memory_gather`` on the index tensors of
                             examples/test_grm.py:203-210.
* ``retriever_*.npz``     -- ``TopKMemoryRetriever.forward`` (weights included).
* ``fusion_*.npz``        -- ``RetrievedStateFusion.forward`` for the four weight-bearing modes.
* ``model_cfg4.npz``      -- samples of the 4-layer ``SegmentMemoryLanguageModel`` forward at config 4
                             (B=8, T=8192, hidden 512, vocab 32768; ``--only model_cfg4``, ~2 min),
                             weights rebuilt from ``seeded_weights.py``.
* ``fusion_cfg3_*.npz``   -- ``RetrievedStateFusion(64, mode)`` as the retrieval configuration builds it
                             (``torch.manual_seed(0)``, default initialisation): weights, a few input rows
                             and the module's outputs on them.
* ``model_cfg1_fp16_archive.npz`` -- the outputs of the same model with the reference's default float16
                             archive storage (weights and inputs are those of ``model_cfg1.npz``).
* ``model_fusion_*.npz``  -- the same model class, smaller (hidden 64, key dim 32, segment 64, four
                             segments), with ``retrieval_fusion_mode`` concat / gate / linear:
                             weights, inputs, outputs and final state.
* ``model_cfg1.npz``      -- ``SegmentRecurrentMemoryModel`` forward on the single-layer
                             adding-problem configuration (weights, inputs, outputs, final
                             state and every segment's routing indices and gates).
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _normalize(x):
    return torch.nn.functional.normalize(x, p=2, dim=-1, eps=1e-6)


def chunk_case(name, seed, B, T, K, H, decay, zero_state=False):
    from grm.core.cuda_ops import _vectorized_chunk_update

    g = torch.Generator().manual_seed(seed)
    k = _normalize(torch.randn(B, T, K, generator=g))
    v = torch.randn(B, T, H, generator=g)
    q = _normalize(torch.randn(B, T, K, generator=g))
    m = torch.zeros(B, H, K) if zero_state else torch.randn(B, H, K, generator=g)
    leaves = [t.clone().requires_grad_(True) for t in (k, v, q, m)]
    hidden, m_out = _vectorized_chunk_update(*leaves, decay)
    loss = hidden.square().mean() + m_out.square().mean()
    loss.backward()
    np.savez_compressed(
        HERE / f"chunk_update_{name}.npz",
        keys=k.numpy(), values=v.numpy(), queries=q.numpy(), memory=m.numpy(), decay=np.float64(decay),
        hidden=hidden.detach().numpy(), memory_out=m_out.detach().numpy(),
        grad_hidden=(2.0 * hidden.detach() / hidden.numel()).numpy(),
        grad_memory_out=(2.0 * m_out.detach() / m_out.numel()).numpy(),
        grad_keys=leaves[0].grad.numpy(), grad_values=leaves[1].grad.numpy(),
        grad_queries=leaves[2].grad.numpy(), grad_memory=leaves[3].grad.numpy(),
    )


def apply_query_case():
    from grm.core.cuda_ops import _fallback_apply_query

    g = torch.Generator().manual_seed(11)
    out = {}
    for tag, mshape, qshape in (("r5", (2, 3, 4, 5, 6), (2, 3, 6)), ("r4", (3, 4, 16, 8), (3, 8))):
        mem = torch.randn(*mshape, generator=g).requires_grad_(True)
        qry = _normalize(torch.randn(*qshape, generator=g)).requires_grad_(True)
        hid = _fallback_apply_query(mem, qry)
        hid.square().mean().backward()
        out.update({
            f"{tag}_memories": mem.detach().numpy(), f"{tag}_queries": qry.detach().numpy(),
            f"{tag}_hidden": hid.detach().numpy(),
            f"{tag}_grad_hidden": (2.0 * hid.detach() / hid.numel()).numpy(),
            f"{tag}_grad_memories": mem.grad.numpy(), f"{tag}_grad_queries": qry.grad.numpy(),
        })
    np.savez_compressed(HERE / "apply_query.npz", **out)


def gather_case():
    from grm.core.cuda_ops import _fallback_batched_memory_gather

    g = torch.Generator().manual_seed(12)
    mem = torch.randn(2, 7, 4, 5, generator=g)
    # the literal index tensors of the reference's own gather test (examples/test_grm.py:203-210)
    idx3 = torch.tensor([[[1, 3], [2, 5], [0, 6]], [[4, 2], [1, 0], [3, 5]]], dtype=torch.long)
    idx2 = torch.tensor([[0, 2, 4], [1, 3, 5]], dtype=torch.long)
    np.savez_compressed(
        HERE / "gather.npz", memories=mem.numpy(), idx3=idx3.numpy(), idx2=idx2.numpy(),
        out3=_fallback_batched_memory_gather(mem, idx3).numpy(),
        out2=_fallback_batched_memory_gather(mem, idx2).numpy(),
    )


def retriever_cases():
    from grm.core.gating_unit import TopKMemoryRetriever

    for name, S, top_k, offset, use_mask in (("topk", 9, 3, 0, False), ("identity", 3, 4, 0, False),
                                            ("causal", 8, 3, 5, False), ("masked", 8, 3, 0, True)):
        torch.manual_seed(21)
        mod = TopKMemoryRetriever(query_dim=6, key_dim=6, hidden_dim=6, retrieval_top_k=top_k, dropout=0.0).eval()
        g = torch.Generator().manual_seed(22)
        query = torch.randn(5, 6, generator=g)
        keys = torch.randn(5, S, 6, generator=g)
        mask = None
        if use_mask:
            mask = torch.ones(5, S, dtype=torch.bool)
            mask[:, 1] = False
            mask[2, 4:] = False
        with torch.no_grad():
            gates, idx, scores = mod(query, keys, segment_offset=offset, attention_mask=mask)
        # margin between the last selected and the best rejected score, to make sure the
        # fixture does not sit on a rounding-sensitive tie
        finite = torch.where(torch.isfinite(scores), scores, torch.full_like(scores, -1e30))
        srt = torch.sort(finite, dim=-1, descending=True).values
        kk = min(top_k, S)
        margin = float((srt[:, kk - 1] - srt[:, kk]).min()) if kk < S else float("inf")
        assert margin > 1e-4, f"retriever fixture {name} has a near-tie (margin {margin})"
        np.savez_compressed(
            HERE / f"retriever_{name}.npz",
            query=query.numpy(), keys=keys.numpy(), segment_offset=np.int64(offset), top_k=np.int64(top_k),
            attention_mask=(mask.numpy() if mask is not None else np.zeros((0,), dtype=bool)),
            w_query=mod.query_projection.weight.detach().numpy(), w_key=mod.key_projection.weight.detach().numpy(),
            gates=gates.numpy(), indices=idx.numpy(), scores=scores.numpy(),
        )


def fusion_cases():
    from grm.core.aggregator import RetrievedStateFusion

    for mode in ("residual", "concat", "gate", "linear"):
        torch.manual_seed(31)
        mod = RetrievedStateFusion(hidden_size=16, retrieval_fusion_mode=mode, dropout=0.0).eval()
        with torch.no_grad():
            mod.layer_norm.weight.uniform_(0.5, 1.5)
            mod.layer_norm.bias.uniform_(-0.5, 0.5)
        g = torch.Generator().manual_seed(32)
        online = torch.randn(7, 16, generator=g)
        retrieved = torch.randn(7, 3, 16, generator=g)
        gates = torch.softmax(torch.randn(7, 3, generator=g), dim=-1)
        with torch.no_grad():
            fused = mod(h_online=online, cached_states=retrieved, gates=gates)
        params = {f"param::{k}": v.detach().numpy() for k, v in mod.state_dict().items()}
        np.savez_compressed(HERE / f"fusion_{mode}.npz", online=online.numpy(), retrieved=retrieved.numpy(),
                            gates=gates.numpy(), fused=fused.numpy(), eps=np.float64(mod.layer_norm.eps), **params)


def fusion_cfg3_cases():
    """The fusion module at the hidden size of the top-k retrieval configuration (d_v = 64, four routes)."""
    from grm.core.aggregator import RetrievedStateFusion

    for mode in ("residual", "concat", "gate", "linear"):
        torch.manual_seed(0)
        mod = RetrievedStateFusion(hidden_size=64, retrieval_fusion_mode=mode, dropout=0.0).eval()
        g = torch.Generator().manual_seed(33)
        online = torch.randn(12, 64, generator=g)
        retrieved = torch.randn(12, 4, 64, generator=g)
        gates = torch.softmax(torch.randn(12, 4, generator=g), dim=-1)
        with torch.no_grad():
            fused = mod(h_online=online, cached_states=retrieved, gates=gates)
        params = {f"param::{k}": v.detach().numpy() for k, v in mod.state_dict().items()}
        np.savez_compressed(HERE / f"fusion_cfg3_{mode}.npz", online=online.numpy(), retrieved=retrieved.numpy(),
                            gates=gates.numpy(), fused=fused.numpy(), eps=np.float64(mod.layer_norm.eps), **params)


def adding_problem_inputs(batch, seq_len, seed):
    """Channel 0 ~ U[0,1); channel 1 marks two positions, one in each half."""
    g = torch.Generator().manual_seed(seed)
    x = torch.zeros(batch, seq_len, 2)
    x[:, :, 0] = torch.rand(batch, seq_len, generator=g)
    half = seq_len // 2
    first = torch.randint(0, half, (batch,), generator=g)
    second = torch.randint(half, seq_len, (batch,), generator=g)
    x[torch.arange(batch), first, 1] = 1.0
    x[torch.arange(batch), second, 1] = 1.0
    return x


def model_cfg1_case():
    from grm.core.paper_grm import SegmentRecurrentMemoryModel

    torch.manual_seed(0)
    model = SegmentRecurrentMemoryModel(
        input_size=2, hidden_size=128, output_size=1, segment_length=128, memory_key_dim=64,
        retrieval_top_k=2, memory_capacity_segments=8, memory_storage_dtype=torch.float32,
        recomputation_ratio=0.0, dropout=0.0, cuda_cpp_debug_fallback=True,
    ).eval()
    x = adding_problem_inputs(2, 512, seed=0)
    routes = []
    original = model._route_chunk

    def recording_route(batch_inputs, segment_keys):
        gates, idx = original(batch_inputs, segment_keys)
        routes.append((gates.clone(), idx.clone()))
        return gates, idx

    model._route_chunk = recording_route
    with torch.no_grad():
        outputs, h_final, memory_final, aux = model(x, reset_memory=True, return_hidden_states=True)
    payload = {f"param::{k}": v.detach().numpy() for k, v in model.state_dict().items()
               if isinstance(v, torch.Tensor) and not k.startswith("memory_bank")}
    for i, (gates, idx) in enumerate(routes):
        payload[f"route{i + 1}_gates"] = gates.numpy()
        payload[f"route{i + 1}_indices"] = idx.numpy()
    np.savez_compressed(
        HERE / "model_cfg1.npz", x=x.numpy(), outputs=outputs.numpy(), h_final=h_final.numpy(),
        memory_final=memory_final.numpy(), hidden_states=aux["hidden_states"].numpy(),
        num_segments=np.int64(aux["num_segments"]), **payload,
    )


def model_cfg1_fp16_archive_case():
    """Config 1 with the reference's DEFAULT archive storage type (float16, grm/core/paper_grm.py:362,139): the
    same seed gives the same weights and inputs as model_cfg1.npz, so only the outputs are stored."""
    from grm.core.paper_grm import SegmentRecurrentMemoryModel

    torch.manual_seed(0)
    model = SegmentRecurrentMemoryModel(
        input_size=2, hidden_size=128, output_size=1, segment_length=128, memory_key_dim=64,
        retrieval_top_k=2, memory_capacity_segments=8, recomputation_ratio=0.0, dropout=0.0,
        cuda_cpp_debug_fallback=True,
    ).eval()
    assert model.memory_bank.memory_storage_dtype == torch.float16
    x = adding_problem_inputs(2, 512, seed=0)
    with torch.no_grad():
        outputs, h_final, memory_final, aux = model(x, reset_memory=True)
    np.savez_compressed(HERE / "model_cfg1_fp16_archive.npz", outputs=outputs.numpy(), h_final=h_final.numpy(),
                        memory_final=memory_final.numpy())


def model_fusion_cases():
    """The single-layer model with each weight-bearing fusion rule, small enough to keep the weights in
    the fixture."""
    from grm.core.paper_grm import SegmentRecurrentMemoryModel

    for seed, mode in enumerate(("concat", "gate", "linear"), start=40):
        torch.manual_seed(seed)
        model = SegmentRecurrentMemoryModel(
            input_size=2, hidden_size=64, output_size=1, segment_length=64, memory_key_dim=32,
            retrieval_top_k=2, memory_capacity_segments=8, memory_storage_dtype=torch.float32,
            recomputation_ratio=0.0, dropout=0.0, retrieval_fusion_mode=mode, cuda_cpp_debug_fallback=True,
        ).eval()
        with torch.no_grad():      # LayerNorm affine away from (1, 0), so that a missing affine shows
            model.aggregator.layer_norm.weight.uniform_(0.5, 1.5)
            model.aggregator.layer_norm.bias.uniform_(-0.5, 0.5)
        x = adding_problem_inputs(2, 256, seed=seed)
        with torch.no_grad():
            outputs, h_final, memory_final, aux = model(x, reset_memory=True, return_hidden_states=True)
        payload = {f"param::{k}": v.detach().numpy() for k, v in model.state_dict().items()
                   if isinstance(v, torch.Tensor) and not k.startswith("memory_bank")}
        np.savez_compressed(
            HERE / f"model_fusion_{mode}.npz", x=x.numpy(), outputs=outputs.numpy(), h_final=h_final.numpy(),
            memory_final=memory_final.numpy(), hidden_states=aux["hidden_states"].numpy(),
            num_segments=np.int64(aux["num_segments"]), **payload,
        )


def model_cfg4_case():
    """4-layer language model of config 4 at full size; only samples of the outputs are stored
    (the weights are rebuilt from seeded_weights.py on both sides)."""
    import time

    from grm.core.multilayer_grm import HierarchicalSegmentMemoryModel
    from grm.utils.train import SegmentMemoryLanguageModel

    sys.path.insert(0, str(HERE))
    from seeded_weights import seeded_state_dict, zipf_token_ids

    vocab, hidden, layers, seq, batch = 32768, 512, 4, 8192, 8
    stack = HierarchicalSegmentMemoryModel(
        hidden, hidden, hidden, num_layers=layers, segment_length=512, memory_key_dim=64, retrieval_top_k=4,
        memory_capacity_segments=16, memory_storage_dtype=torch.float32, recomputation_ratio=0.0, dropout=0.0,
        cuda_cpp_debug_fallback=True)
    model = SegmentMemoryLanguageModel(stack, vocab_size=vocab, embed_dim=hidden).eval()
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()
              if isinstance(v, torch.Tensor) and "memory_bank" not in k}
    missing = model.load_state_dict(seeded_state_dict(shapes), strict=False)
    assert not missing.unexpected_keys
    ids = zipf_token_ids(batch, seq, vocab, 1.1, seed=0)
    torch.set_num_threads(8)
    t0 = time.time()
    with torch.no_grad():
        logits, h_final, c_final, aux = model(ids, reset_memory=True)
    print(f"config-4 reference forward: {time.time() - t0:.1f} s")
    positions = torch.tensor([0, 1, 511, 512, 513, 1023, 1024, 2047, 4095, 4096, 6000, 8190, 8191])
    np.savez_compressed(
        HERE / "model_cfg4.npz",
        positions=positions.numpy(), logits=logits[:, positions, :256].numpy(),
        logit_row_norms=logits[:, positions].norm(dim=-1).numpy(),
        c_final=c_final[:, :, :16, :16].numpy(), c_final_norm=c_final.flatten(2).norm(dim=-1).numpy(),
        num_segments=np.int64(aux["num_segments"]),
        shape_names=np.array(list(shapes.keys())), shape_dims=np.array([str(v) for v in shapes.values()]),
    )


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--reference", type=Path,
                        default=Path(os.environ.get("GRM_REFERENCE_ROOT", "") or HERE.parents[2] / "reference"),
                        help="reference checkout (default: $GRM_REFERENCE_ROOT, else a `reference` folder beside the repository)")
    parser.add_argument("--only", default="", help="generate only this fixture (e.g. model_cfg4)")
    args = parser.parse_args(argv)
    sys.dont_write_bytecode = True
    sys.path.insert(0, str(args.reference))
    torch.set_num_threads(1)
    if args.only == "model_cfg4":
        model_cfg4_case()
        return 0
    if args.only == "model_fusion":
        model_fusion_cases()
        return 0
    if args.only == "model_cfg1_fp16_archive":
        model_cfg1_fp16_archive_case()
        return 0
    if args.only == "fusion_cfg3":
        fusion_cfg3_cases()
        return 0
    chunk_case("small", 1, B=2, T=8, K=8, H=16, decay=0.97)        # shape of examples/test_grm.py:29-37
    chunk_case("ragged", 2, B=3, T=67, K=6, H=5, decay=0.9)
    chunk_case("cfg1", 3, B=2, T=128, K=64, H=128, decay=0.97, zero_state=True)
    chunk_case("long", 4, B=1, T=300, K=32, H=48, decay=0.999)
    apply_query_case()
    gather_case()
    retriever_cases()
    fusion_cases()
    fusion_cfg3_cases()
    model_cfg1_case()
    model_cfg1_fp16_archive_case()
    model_fusion_cases()
    total = sum(p.stat().st_size for p in HERE.glob("*.npz"))
    print(f"wrote {len(list(HERE.glob('*.npz')))} fixtures, {total / 1024:.0f} KiB")
    return 0


if __name__ == "__main__":
    sys.exit(main())
