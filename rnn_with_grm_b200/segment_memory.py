"""The callers on either side of the kernels: archive, segment loop, stacked model.

``SegmentMemoryRunner.forward`` is the reference's ``SegmentRecurrentMemoryModel.forward``
(grm/core/paper_grm.py:647-747) driven by this engine's kernels, restructured in ways that leave the
results unchanged:

* the archive is a preallocated device ring ``[B, capacity, H, K]`` written in place, instead of a
  deque of tensors that is re-stacked and permuted for every segment (paper_grm.py:135-146, 227-228);
  it also keeps the routing keys of its segments (projected once) and, for bf16 activations, a bf16
  copy of the ring;
* retrieval never materialises the gathered ``[B, C, R, H, K]`` tensor of paper_grm.py:229-234:
  either one kernel reads the selected matrices straight from the ring
  (``torch.ops.grmx.retrieve_fuse``), or, with per-token routing, the queries of a segment are
  applied to all archived matrices with one batched GEMM and ``torch.ops.grmx.select_fuse`` picks,
  weights, adds and normalises;
* everything that depends on the layer input alone (projections, summaries, routing keys) is
  computed for the whole sequence before the loop;
* bf16 activations over whole segments that fit the archive run without a loop at all: one scan
  launch leaves the state at every segment end in the ring, then routing, apply-query and selection
  run once for all tokens (``_run_whole_sequence``); the retrieval of a segment never feeds back into
  the recurrence, and a token of segment i sees only the slots that were archived before it.

Parameters are taken by the names of the reference model's ``state_dict`` so a checkpoint of
the reference loads as is.  Projections and the weight-bearing fusion rules are plain
``torch.nn.functional`` calls (cuBLAS); everything on the memory path goes through
``cuda_ops`` / ``torch.ops.grmx``.  CUDA only, inference only (no autograd through the ring).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from . import cuda_ops

FUSE_RETRIEVED, FUSE_CONTRIB, FUSE_RESIDUAL_LN = 0, 1, 2


class SegmentMemoryArchive:
    """Bounded FIFO of segment-end memories and segment summaries, resident on the device.

    Same contract as the reference's ``_BatchMemoryArchive`` (paper_grm.py:31-44): at most
    ``capacity`` segments, the oldest evicted first, and routing indices are positions in
    the current FIFO order (0 = oldest).
    """

    def __init__(self, batch: int, capacity: int, hidden: int, key_dim: int, summary_dim: int, device,
                 storage_dtype: torch.dtype = torch.float32):
        self.capacity = int(capacity)
        # The reference keeps archived memories and summaries in ``memory_storage_dtype`` and widens them to
        # fp32 when it reads them (paper_grm.py:139-140, 227).  The ring itself is fp32 (the kernels read it
        # as it is); with another storage type every value goes through that type once, on its way in.
        self.storage_dtype = storage_dtype
        if torch.device(device).type == "cuda" and not cuda_ops.load_grm_cuda_extension():
            raise RuntimeError("the grm_cuda extension is not loaded: " +
                               str(cuda_ops.get_grm_cuda_runtime_status().get("load_error")))
        self.memories = torch.empty(batch, self.capacity, hidden, key_dim, device=device, dtype=torch.float32)
        self.summaries = torch.empty(batch, self.capacity, summary_dim, device=device, dtype=torch.float32)
        # the summaries as the router scores them (projected once, when the segment is archived)
        self.route_keys: Optional[Tensor] = None
        # bf16 copy of ``memories`` for retrieval with bf16 activations, written by the same kernel
        self.memories_bf16: Optional[Tensor] = None
        self.count = 0      # segments held
        self.head = 0       # physical slot of the oldest segment
        self.total_pushed = 0

    def _route_key_buffer(self, dim: int) -> Tensor:
        if self.route_keys is None or self.route_keys.shape[-1] != dim:
            if self.count > 0:
                raise RuntimeError("route keys must be pushed with every segment or with none")
            self.route_keys = torch.empty(self.summaries.shape[0], self.capacity, dim,
                                          device=self.summaries.device, dtype=torch.float32)
        return self.route_keys

    def write_ahead(self, summaries: Tensor, route_keys: Tensor) -> bool:
        """Store the summaries and routing keys ``[B, n, D]`` of the next ``n`` pushes with one copy
        each.  Only when those pushes evict nothing and their slots do not wrap: the slots are then
        free and stay invisible (beyond ``count``) until their push.  Returns whether it was done; if
        so, the pushes pass ``summary=None``."""
        n = summaries.shape[1]
        first = self.head + self.count
        if n == 0 or first + n > self.capacity:
            return False
        self.summaries[:, first:first + n].copy_(summaries)
        self._route_key_buffer(route_keys.shape[-1])[:, first:first + n].copy_(route_keys)
        return True

    def note_pushed(self, n: int) -> None:
        """``n`` segments were written into the slots after the held ones (by the scan itself)."""
        if self.head != 0 or self.count + n > self.capacity:
            raise RuntimeError("slots written in place must not wrap or evict")
        self.count += n
        self.total_pushed += n

    def keep_bf16_copy(self) -> None:
        if self.memories_bf16 is None:
            self.memories_bf16 = self.memories.to(torch.bfloat16)

    def as_stored(self, t: Tensor) -> Tensor:
        """``t`` as it reads back from the archive: rounded through the storage type, fp32."""
        if self.storage_dtype == torch.float32:
            return t.float()
        return t.to(self.storage_dtype).float()

    def push(self, memory: Tensor, summary: Optional[Tensor], route_key: Optional[Tensor] = None) -> None:
        slot = (self.head + self.count) % self.capacity
        if self.storage_dtype != torch.float32:
            memory = self.as_stored(memory)
            summary = None if summary is None else self.as_stored(summary)
        if memory.is_cuda and memory.dtype == torch.float32:
            torch.ops.grmx.archive_push(memory, self.memories, self.memories_bf16, slot)
        else:
            self.memories[:, slot].copy_(memory)
            if self.memories_bf16 is not None:
                self.memories_bf16[:, slot].copy_(memory)
        if summary is not None:
            self.summaries[:, slot].copy_(summary)
        if summary is not None and route_key is not None:
            self._route_key_buffer(route_key.shape[-1])[:, slot].copy_(route_key)
        if self.count < self.capacity:
            self.count += 1
        else:
            self.head = (self.head + 1) % self.capacity
        self.total_pushed += 1

    def ordered_summaries(self) -> Tensor:
        """``[B, count, D]`` in FIFO order."""
        if self.head == 0:
            return self.summaries[:, : self.count]
        order = (torch.arange(self.count, device=self.summaries.device) + self.head) % self.capacity
        return self.summaries.index_select(1, order)

    # ---- checkpoint / resume in the reference's layout ----------------------------------------

    def get_extra_state(self) -> dict:
        """The archived segments as the reference's ``SegmentMemoryArchive.get_extra_state`` lays them
        out (paper_grm.py:98-114): per batch size, the memories ``[B, H, K]`` and summaries ``[B, D]``
        oldest first.  ``checkpoints`` (inputs kept for selective recomputation, which this engine does
        not do) is an empty list."""
        slots = [(self.head + i) % self.capacity for i in range(self.count)]
        batch = int(self.memories.shape[0])
        return {"groups": {batch: {"memories": [self.memories[:, s].clone() for s in slots],
                                   "summaries": [self.summaries[:, s].clone() for s in slots],
                                   "checkpoints": []}}}

    def set_extra_state(self, state: Optional[dict]) -> None:
        """Refill the ring from a state saved by this class or by the reference (paper_grm.py:116-133).
        Only the group of this archive's batch size is read; more segments than the capacity keep the
        newest.  The routing keys are left for the runner to project again."""
        self.count = self.head = 0
        self.route_keys = None
        self.memories_bf16 = None
        groups = {} if state is None else state.get("groups", {})
        batch = int(self.memories.shape[0])
        group = groups.get(batch, groups.get(str(batch)))
        if group is None:
            return
        memories, summaries = list(group.get("memories", [])), list(group.get("summaries", []))
        if len(memories) != len(summaries):
            raise ValueError("extra state holds a different number of memories and summaries")
        for memory, summary in zip(memories, summaries):
            if tuple(memory.shape) != tuple(self.memories.shape[0:1] + self.memories.shape[2:]):
                raise ValueError(f"archived memory of shape {tuple(memory.shape)} does not fit this archive")
            device = self.memories.device
            self.push(memory.to(device=device, dtype=torch.float32).contiguous(), summary.to(device=device))
            self.total_pushed -= 1      # restoring is not pushing; the reference keeps this counter in its state_dict

    def set_route_keys(self, keys: Tensor) -> None:
        """Routing keys ``[B, count, D_route]`` of the archived segments, oldest first."""
        if keys.shape[1] != self.count:
            raise ValueError("one routing key per archived segment")
        buffer = torch.empty(self.summaries.shape[0], self.capacity, keys.shape[-1], device=self.summaries.device,
                             dtype=torch.float32)
        slots = (torch.arange(self.count, device=buffer.device) + self.head) % self.capacity
        buffer.index_copy_(1, slots, keys.to(torch.float32))
        self.route_keys = buffer

    def ordered_route_keys(self) -> Tensor:
        """``[B, count, D_route]`` in FIFO order."""
        if self.head == 0:
            return self.route_keys[:, : self.count]
        order = (torch.arange(self.count, device=self.route_keys.device) + self.head) % self.capacity
        return self.route_keys.index_select(1, order)

    def physical_indices(self, indices: Tensor) -> Tensor:
        """FIFO positions -> slots of ``self.memories`` (empty slots, -1, stay -1)."""
        if self.head == 0:
            return indices
        return torch.where(indices >= 0, (indices + self.head) % self.capacity, indices)


def _check_errors_if_asked() -> None:
    """With ``GRMX_CHECK_ERRORS`` set, raise if a kernel of the pass reported a failure through the device
    error word (``cuda_ops.check_device_errors``); never during stream capture, where nothing may wait."""
    if cuda_ops._checking_each_call() and not torch.cuda.is_current_stream_capturing():
        cuda_ops.check_device_errors()


def _linear(x: Tensor, params: Dict[str, Tensor], name: str) -> Tensor:
    return F.linear(x, params[f"{name}.weight"], params.get(f"{name}.bias"))


def _l2_normalized(t: Tensor) -> Tensor:
    """``F.normalize(t, p=2, dim=-1, eps=1e-6)`` (paper_grm.py:491-493) in one pass over ``t``."""
    per16 = 16 // t.element_size()
    K = t.shape[-1]
    if t.is_cuda and t.dtype in (torch.float32, torch.bfloat16) and K % per16 == 0 and K // per16 <= 128:
        return torch.ops.grmx.l2_normalize(t, 1e-6, False)
    return F.normalize(t, p=2, dim=-1, eps=1e-6)


class SegmentMemoryRunner:
    """One segment-memory layer: scan -> route -> retrieve + fuse -> output projection."""

    def __init__(self, params: Dict[str, Tensor], *, segment_length: int, retrieval_top_k: int,
                 memory_capacity_segments: int, memory_decay: float = 0.97,
                 retrieval_fusion_mode: str = "residual", memory_initialization_mode: str = "checkpoint",
                 use_layer_norm: bool = True, layer_norm_eps: float = 1e-5, temperature: float = 1.0,
                 memory_storage_dtype: torch.dtype = torch.float16):
        if retrieval_fusion_mode not in ("residual", "concat", "gate", "linear"):
            raise ValueError(f"Unknown retrieval_fusion_mode: {retrieval_fusion_mode}")
        self.p = params
        self.segment_length = int(segment_length)
        self.top_k = int(retrieval_top_k)
        self.capacity = int(memory_capacity_segments)
        self.decay = float(memory_decay)
        self.mode = retrieval_fusion_mode
        self.init_mode = memory_initialization_mode
        self.use_layer_norm = use_layer_norm
        self.eps = float(layer_norm_eps)
        self.temperature = float(temperature)
        # type the archive keeps memories and summaries in; float16 is the reference's default (paper_grm.py:362)
        self.storage_dtype = memory_storage_dtype
        self.hidden = params["memory_cell.value_proj.weight"].shape[0]
        self.key_dim = params["memory_cell.key_proj.weight"].shape[0]
        self.input_size = params["memory_cell.key_proj.weight"].shape[1]
        self.route_dim = params["gating_unit.query_projection.weight"].shape[0]
        self.archive: Optional[SegmentMemoryArchive] = None
        self.dense_retrieval = True    # False: always gather the selected matrices (retrieve_fuse kernel)
        # Per-token routing scores every token against at most ``capacity`` summaries.  Folded, the
        # query projection is applied to those few projected keys (``[S, route_dim] x [route_dim, D]``)
        # and the tokens are scored unprojected: the ``[B*T, D] x [D, route_dim]`` fp32 GEMM disappears.
        # The scores are the same sums associated differently, equal to fp32 rounding.
        # Set it before the first call (the archive keeps the keys in the form they were pushed in).
        self.fold_routing_projection = True
        self.parallel_summaries = True     # whole-sequence form: summaries and routing keys beside the scan
        self._side_streams: Dict[str, torch.cuda.Stream] = {}
        # Whole segments of bf16 activations that fit the archive without evicting run as one scan
        # launch plus one routing / selection pass for all tokens (see _run_whole_sequence).
        self.fuse_segments = True
        self.max_state_bytes = 1 << 30      # candidate states held at a time by the whole-sequence form
        # bf16 activations with a 64-wide key: the retrieval runs on the tensor cores straight from the bf16
        # ring (``torch.ops.grmx.retrieve_fuse_tc``), one accumulated product per chosen slot and token tile,
        # and neither gathered matrices nor candidate states exist.  False: the batched GEMM over all
        # candidates followed by ``select_fuse``.
        self.tensor_core_retrieval = True
        # key and query projections with the normalisation in the epilogue (see _keys_and_queries)
        self.fused_projection = True
        self._stacked_kq = None
        self._route_query_weight: Optional[Tensor] = None
        self._fp32_cache: Dict[str, Tuple[Tensor, Tensor, int]] = {}
        self._visible_cache: Dict[Tuple[int, int, str], Tensor] = {}

    def clear_memory(self) -> None:
        self.archive = None

    def get_extra_state(self) -> dict:
        """The archive in the reference's checkpoint layout (see ``SegmentMemoryArchive.get_extra_state``)."""
        return {"groups": {}} if self.archive is None else self.archive.get_extra_state()

    def set_extra_state(self, state: Optional[dict], device=None) -> None:
        """Resume from a saved archive: the next ``forward(..., reset_memory=False)`` retrieves from it."""
        groups = {} if state is None else state.get("groups", {})
        if not groups:
            self.archive = None
            return
        batch, group = next(iter(groups.items()))
        memories = group.get("memories", [])
        if not memories:
            self.archive = None
            return
        device = memories[0].device if device is None else torch.device(device)
        self.archive = SegmentMemoryArchive(int(batch), self.capacity, self.hidden, self.key_dim, self.input_size, device,
                                            self.storage_dtype)
        self.archive.set_extra_state({"groups": {int(batch): group}})

    def _keys_and_queries(self, x: Tensor) -> Tuple[Tensor, Tensor]:
        """``F.normalize(key_proj(x))`` and ``F.normalize(query_proj(x))`` (paper_grm.py:491-493).  bf16
        activations with a 64-wide key take one pass over ``x``: both projections as one tensor-core product
        with the normalisation in its epilogue (``torch.ops.grmx.project_normalize``); otherwise two GEMMs and
        the one-pass normalisation kernel."""
        wk, wq = self.p["memory_cell.key_proj.weight"], self.p["memory_cell.query_proj.weight"]
        D = x.shape[-1]
        if (self.fused_projection and x.is_cuda and x.dtype == torch.bfloat16 and wk.dtype == torch.bfloat16
                and self.key_dim == 64 and D % 64 == 0 and D <= 512):
            cached = self._stacked_kq
            versions = (wk._version, wq._version)
            if cached is None or cached[0] is not wk or cached[1] is not wq or cached[2] != versions:
                bk, bq = self.p.get("memory_cell.key_proj.bias"), self.p.get("memory_cell.query_proj.bias")
                bias = None
                if bk is not None or bq is not None:
                    zero = torch.zeros(self.key_dim, device=x.device)
                    bias = torch.cat([zero if bk is None else bk.float(), zero if bq is None else bq.float()]).contiguous()
                cached = (wk, wq, versions, torch.cat([wk, wq], dim=0).contiguous(), bias)
                self._stacked_kq = cached
            k, q = torch.ops.grmx.project_normalize(x, cached[3], cached[4], 1e-6)
            return k, q
        return (_l2_normalized(_linear(x, self.p, "memory_cell.key_proj")),
                _l2_normalized(_linear(x, self.p, "memory_cell.query_proj")))

    def _fp32_param(self, name: str) -> Optional[Tensor]:
        """The parameter as the kernels read it (fp32), converted once per parameter tensor."""
        t = self.p.get(name)
        if t is None or t.dtype == torch.float32:
            return t
        cached = self._fp32_cache.get(name)
        if cached is None or cached[0] is not t or cached[2] != t._version:
            cached = (t, t.float(), t._version)
            self._fp32_cache[name] = cached
        return cached[1]

    def _visible_counts(self, queries: int, count: int, device) -> Tensor:
        key = (queries, count, str(device))
        t = self._visible_cache.get(key)
        if t is None:
            t = torch.full((queries,), count, device=device, dtype=torch.int32)
            self._visible_cache[key] = t
        return t

    # ---- pieces of one segment -------------------------------------------------------------

    def _side_stream(self, device) -> "torch.cuda.Stream":
        key = str(device)
        stream = self._side_streams.get(key)
        if stream is None:
            stream = torch.cuda.Stream(device=device)
            self._side_streams[key] = stream
        return stream

    def _route_keys(self, summaries: Tensor) -> Tensor:
        """Segment summaries ``[B, n, D]`` as the router scores them (paper_grm.py:566-570: bias-free
        key projection).  In the folded form the query projection is applied here as well:
        ``(x Wq^T) . (s Wk^T) == x . ((s Wk^T) Wq)``, so the few keys are projected back instead of
        every token forward."""
        keys = F.linear(summaries, self._route_key_weight)
        if self._route_query_weight is not None:
            keys = torch.matmul(keys, self._route_query_weight)
        return keys

    def _route(self, route_q: Tensor, keys: Tensor, visible: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
        """``route_q``: the projected routing queries, or (folded form) the fp32 layer input itself.
        ``visible``: per query, how many of the leading keys it may choose from (all if None)."""
        # paper_grm.py:571-589: scale 1/sqrt(route_dim), top-k, softmax over the selected scores
        gates, indices, _ = torch.ops.grmx.topk_route(route_q, keys, visible, self.top_k,
                                                      1.0 / math.sqrt(self.route_dim), self.temperature, False)
        return gates, indices

    def _dense_states(self, q_t: Tensor) -> Tensor:
        """Every archived matrix of a batch row applied to every query of the segment: ``[B, C, count, H]``.

        With per-token routing all tokens of a segment pick among the same ``count`` archived
        matrices, so applying the query to all of them is one small batched GEMM
        (``[C, K] x [K, count*H]`` per batch row, cuBLAS) and the selection becomes a pick of
        H-vectors (``torch.ops.grmx.select_fuse``): ``count*H*K`` reads per batch row instead of
        ``C*R*H*K`` (config 4: 15 candidates against 512 tokens x 4 routes).  Same result as gather +
        apply-query up to summation order.
        """
        archive = self.archive
        B, C, _ = q_t.shape
        ring = archive.memories_bf16 if q_t.dtype == torch.bfloat16 and archive.memories_bf16 is not None \
            else archive.memories
        mem = ring[:, : archive.count] if archive.head == 0 else ring.index_select(
            1, (torch.arange(archive.count, device=q_t.device) + archive.head) % archive.capacity)
        mem = mem.reshape(B, archive.count * self.hidden, self.key_dim).to(q_t.dtype)
        return torch.matmul(q_t, mem.transpose(1, 2)).view(B, C, archive.count, self.hidden)

    def _tc_retrieval_applies(self, q: Tensor, routes: int) -> bool:
        archive = self.archive
        return (self.tensor_core_retrieval and q.is_cuda and q.dtype == torch.bfloat16 and archive is not None
                and archive.memories_bf16 is not None and self.key_dim == 64 and self.hidden % 64 == 0
                and self.hidden <= 512 and archive.capacity <= 32 and 1 <= routes <= 8)

    def _retrieve_and_fuse(self, q_n: Tensor, h_online: Tensor, gates: Tensor, indices: Tensor) -> Tensor:
        """``q_n``: the segment's normalised queries (paper_grm.py:301,312 recompute the same values)."""
        archive = self.archive
        ln_w = self._fp32_param("aggregator.layer_norm.weight") if self.use_layer_norm else None
        ln_b = self._fp32_param("aggregator.layer_norm.bias") if self.use_layer_norm else None
        plain_residual = (self.mode == "residual" and self.use_layer_norm
                          and "aggregator.output_projection.weight" not in self.p)
        if self._tc_retrieval_applies(q_n, indices.shape[2]):
            phys = archive.physical_indices(indices)
            if plain_residual:
                return torch.ops.grmx.retrieve_fuse_tc(archive.memories_bf16, phys, gates, q_n, h_online, ln_w, ln_b,
                                                       self.eps, FUSE_RESIDUAL_LN)
            contrib = torch.ops.grmx.retrieve_fuse_tc(archive.memories_bf16, phys, gates, q_n, None, None, None,
                                                      self.eps, FUSE_CONTRIB)
            return self._fuse_rule(h_online, contrib)
        # queries x routes against candidates: the dense form reads every candidate once per batch row
        dense = self.dense_retrieval and indices.shape[1] * indices.shape[2] >= 4 * archive.count
        if dense:
            states = self._dense_states(q_n)
            if plain_residual:
                return torch.ops.grmx.select_fuse(states, indices, gates, h_online.to(states.dtype), ln_w, ln_b,
                                                  self.eps, FUSE_RESIDUAL_LN).to(h_online.dtype)
            contrib = torch.ops.grmx.select_fuse(states, indices, gates, None, None, None, self.eps,
                                                 FUSE_CONTRIB).to(h_online.dtype)
        else:
            q_t = q_n.float()
            phys = archive.physical_indices(indices)
            if plain_residual:
                fused = torch.ops.grmx.retrieve_fuse(archive.memories, phys, gates, q_t, h_online.float(), ln_w, ln_b,
                                                     self.eps, FUSE_RESIDUAL_LN)
                return fused.to(h_online.dtype)
            contrib = torch.ops.grmx.retrieve_fuse(archive.memories, phys, gates, q_t, None, None, None, self.eps,
                                                   FUSE_CONTRIB).to(h_online.dtype)
        return self._fuse_rule(h_online, contrib)

    def _fuse_rule(self, h_online: Tensor, contrib: Tensor) -> Tensor:
        """The fusion rules other than the plain residual one, on the gate-weighted contribution."""
        # aggregator.py:116-145
        if self.mode == "residual":
            fused = h_online + contrib
            if "aggregator.output_projection.weight" in self.p:
                fused = _linear(fused, self.p, "aggregator.output_projection")
        elif self.mode == "concat":
            fused = _linear(torch.cat([h_online, contrib], dim=-1), self.p, "aggregator.output_projection")
        elif self.mode == "gate":
            gate = torch.sigmoid(_linear(torch.cat([h_online, contrib], dim=-1), self.p, "aggregator.gate_projection"))
            fused = gate * h_online + (1.0 - gate) * contrib
        else:
            fused = _linear(h_online, self.p, "aggregator.online_projection") + \
                _linear(contrib, self.p, "aggregator.memory_projection")
        if self.use_layer_norm:
            fused = F.layer_norm(fused, (self.hidden,), self.p.get("aggregator.layer_norm.weight"),
                                 self.p.get("aggregator.layer_norm.bias"), self.eps)
        return fused

    # ---- the segment loop ------------------------------------------------------------------

    @torch.no_grad()
    def forward(self, x_seq: Tensor, c_init: Optional[Tensor] = None, reset_memory: bool = False,
                return_routes: bool = False):
        """``x_seq [B, T, D]`` -> ``(outputs [B, T, out], h_final [B, H], memory_final [B, H, K], aux)``."""
        B, T, _ = x_seq.shape
        L = self.segment_length
        if self.whole_sequence_applies(x_seq, reset_memory):
            result = self._run_whole_sequence(x_seq, c_init, reset_memory, return_routes)
        elif T > 0 and T % L == 0:
            x_sm = x_seq.reshape(B, T // L, L, -1).transpose(0, 1).contiguous()
            out, last_hidden, memory, aux = self._run(x_sm, True, c_init, reset_memory, return_routes)
            result = out.transpose(0, 1).reshape(B, T, -1), last_hidden, memory, aux
        else:
            result = self._run(x_seq, False, c_init, reset_memory, return_routes)
        _check_errors_if_asked()
        return result

    @torch.no_grad()
    def forward_segment_major(self, x_sm: Tensor, c_init: Optional[Tensor] = None, reset_memory: bool = False,
                              return_routes: bool = False):
        """The same on ``x_sm [T/L, B, L, D]`` (segment ``i`` of every batch row contiguous), outputs in
        the same layout.  The kernels take one segment of all batch rows at a time, so a caller that
        keeps this layout across layers saves the two transpositions per layer."""
        if x_sm.dim() != 4 or x_sm.shape[2] != self.segment_length:
            raise ValueError("expected [segments, B, segment_length, D]")
        return self._run(x_sm.contiguous(), True, c_init, reset_memory, return_routes)

    # ---- all segments at once ------------------------------------------------------------------
    #
    # The retrieval of a segment never feeds back into the recurrence: the memory update reads the
    # keys and values of the layer input only (paper_grm.py:491-523), and the fused hidden state goes
    # to the output projection.  What is sequential in the segments is the scan state alone.  So one
    # scan launch runs over the whole sequence and leaves the state at every segment end in the
    # archive ring, and routing, dense apply-query and selection follow for all tokens at once: a
    # token of segment i may choose among the first count0 + i slots only, the later slots (already
    # written) stay invisible to it.

    def whole_sequence_applies(self, x: Tensor, reset_memory: bool) -> bool:
        L = self.segment_length
        B, T = x.shape[0], x.shape[1]
        if not (self.fuse_segments and x.is_cuda and x.dtype == torch.bfloat16 and T > 0 and T % L == 0 and L % 128 == 0):
            return False
        if self.init_mode != "checkpoint" or not self.dense_retrieval or self.capacity > 16:
            return False
        if self.key_dim % 64 or self.hidden % 64 or self.key_dim > 1024 or self.hidden > 1024:
            return False
        held = 0
        if self.archive is not None and not reset_memory:
            if self.archive.head != 0 or self.archive.memories.shape[0] != B:
                return False
            held = self.archive.count
        return held + T // L <= self.capacity

    def _run_whole_sequence(self, x: Tensor, c_init: Optional[Tensor], reset_memory: bool, return_routes: bool):
        B, T, _ = x.shape
        L = self.segment_length
        n_seg = T // L
        if reset_memory:
            self.clear_memory()
        if self.archive is None:
            self.archive = SegmentMemoryArchive(B, self.capacity, self.hidden, self.key_dim, self.input_size, x.device,
                                                self.storage_dtype)
        archive = self.archive
        archive.keep_bf16_copy()
        memory = c_init.float() if c_init is not None else torch.zeros(B, self.hidden, self.key_dim, device=x.device,
                                                                       dtype=torch.float32)
        route_q_weight = self._fp32_param("gating_unit.query_projection.weight")
        self._route_key_weight = self._fp32_param("gating_unit.key_projection.weight")
        fold = self.fold_routing_projection and self.input_size <= 2 * self.route_dim
        self._route_query_weight = route_q_weight if fold else None
        if archive.count > 0 and archive.route_keys is None:       # an archive restored from a saved state
            archive.set_route_keys(self._route_keys(archive.ordered_summaries()))
        first = archive.count                                        # head == 0 here
        # The segment summaries, their routing keys (a mean and two small GEMMs, all of them far from filling
        # the GPU) and the routing depend on the layer input only: they run on a stream of their own beside
        # the projections and the scan, and the retrieval waits for them.
        main = torch.cuda.current_stream(x.device)
        side = self._side_stream(x.device) if self.parallel_summaries else main
        if side is not main:
            side.wait_stream(main)
        with torch.cuda.stream(side):
            summaries = archive.as_stored(x.reshape(B, n_seg, L, -1).mean(dim=2, dtype=torch.float32))
            new_keys = self._route_keys(summaries)
            if not archive.write_ahead(summaries, new_keys):
                raise RuntimeError("the archive cannot take the segments of this call without evicting")
            # the routing itself needs the layer input and the keys only, nothing of the scan
            held = first + n_seg
            gates = indices = None
            if held > 1 or first > 0:
                visible = self._visible_ramp(T, L, first, x.device)      # tokens of segment i see first + i slots
                route_q = x if fold else F.linear(x.float(), route_q_weight)
                gates, indices = self._route(route_q, archive.route_keys, visible)
        k, q = self._keys_and_queries(x)
        v = _linear(x, self.p, "memory_cell.value_proj")
        hidden, memory = torch.ops.grmx.chunk_scan_segments(k, v, q, memory, self.decay, archive.memories, first, L)
        if side is not main:
            main.wait_stream(side)       # what the side stream allocated stays referenced until the end of this call
        archive.note_pushed(n_seg)
        if archive.storage_dtype != torch.float32:      # the states the scan left in the ring, as the archive stores them
            archive.memories[:, first:first + n_seg] = archive.as_stored(archive.memories[:, first:first + n_seg])
        archive.memories_bf16[:, first:first + n_seg].copy_(archive.memories[:, first:first + n_seg])
        routes = []
        if held > 1 or first > 0:
            ring = archive.memories_bf16[:, :held].reshape(B, held * self.hidden, self.key_dim)
            ln_w = self._fp32_param("aggregator.layer_norm.weight") if self.use_layer_norm else None
            ln_b = self._fp32_param("aggregator.layer_norm.bias") if self.use_layer_norm else None
            plain_residual = (self.mode == "residual" and self.use_layer_norm
                              and "aggregator.output_projection.weight" not in self.p)
            tensor_core = self._tc_retrieval_applies(q, indices.shape[2])
            # the candidate states of a block of segments at a time, at most ~1 GiB of them (one block at
            # config 4; four blocks, each with only the candidates its last segment sees, compute 40 %
            # less but measured slower: 5.24 against 4.92 ms)
            per_segment = B * L * held * self.hidden * 2
            block = max(1, min(n_seg, self.max_state_bytes // max(per_segment, 1)))
            pieces = []
            if tensor_core:
                # all tokens at once, straight from the bf16 ring: a token's routes name slots below its own
                # visible count only, so the later slots (already written by the scan) stay untouched
                if plain_residual:
                    pieces.append(torch.ops.grmx.retrieve_fuse_tc(archive.memories_bf16, indices, gates, q, hidden, ln_w,
                                                                  ln_b, self.eps, FUSE_RESIDUAL_LN))
                else:
                    contrib = torch.ops.grmx.retrieve_fuse_tc(archive.memories_bf16, indices, gates, q, None, None, None,
                                                              self.eps, FUSE_CONTRIB)
                    pieces.append(self._fuse_rule(hidden, contrib))
            for s0 in range(0, n_seg if not tensor_core else 0, block):
                s1 = min(s0 + block, n_seg)
                tok = slice(s0 * L, s1 * L)
                slots = first + s1 - 1                                # the last segment of the block sees this many
                if slots == 0:
                    pieces.append(hidden[:, tok])
                    continue
                states = torch.matmul(q[:, tok], ring[:, : slots * self.hidden].transpose(1, 2)).view(
                    B, (s1 - s0) * L, slots, self.hidden)
                if plain_residual:
                    pieces.append(torch.ops.grmx.select_fuse(states, indices[:, tok].contiguous(), gates[:, tok].contiguous(),
                                                             hidden[:, tok].contiguous(), ln_w, ln_b, self.eps,
                                                             FUSE_RESIDUAL_LN))
                else:
                    contrib = torch.ops.grmx.select_fuse(states, indices[:, tok].contiguous(), gates[:, tok].contiguous(),
                                                         None, None, None, self.eps, FUSE_CONTRIB)
                    pieces.append(self._fuse_rule(hidden[:, tok], contrib))
            fused = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=1)
            if first == 0 and not plain_residual:
                # the first segment saw an empty archive: no fusion at all for it (paper_grm.py:620-621;
                # the plain residual kernel passes such tokens through by itself)
                fused = torch.cat([hidden[:, :L], fused[:, L:]], dim=1)
            if return_routes:
                for i in range(n_seg):
                    if first + i > 0:
                        routes.append((gates[:, i * L:(i + 1) * L], indices[:, i * L:(i + 1) * L]))
        else:
            fused = hidden
        last_hidden = fused[:, -1]
        out = _linear(fused, self.p, "output_proj")
        aux = {"num_segments": archive.count, "total_pushed": archive.total_pushed}
        if return_routes:
            aux["routes"] = routes
        return out, last_hidden, memory, aux

    def _visible_ramp(self, T: int, L: int, first: int, device) -> Tensor:
        key = ("ramp", T, L, first, str(device))
        t = self._visible_cache.get(key)
        if t is None:
            t = (torch.arange(T, device=device, dtype=torch.int32) // L + first).to(torch.int32)
            self._visible_cache[key] = t
        return t

    def _run(self, x: Tensor, segment_major: bool, c_init: Optional[Tensor], reset_memory: bool,
             return_routes: bool):
        """``x``: ``[n, B, L, D]`` when ``segment_major`` (all segments full), else ``[B, T, D]``."""
        if x.device.type != "cuda":
            raise RuntimeError("SegmentMemoryRunner needs CUDA tensors; this engine has no CPU path")
        L = self.segment_length
        if segment_major:
            n_seg, B = x.shape[0], x.shape[1]
            bounds = [(i * L, (i + 1) * L) for i in range(n_seg)]
        else:
            B, T, _ = x.shape
            bounds = [(s0, min(s0 + L, T)) for s0 in range(0, T, L)]
        if reset_memory:
            self.clear_memory()
        if self.archive is None:
            self.archive = SegmentMemoryArchive(B, self.capacity, self.hidden, self.key_dim, self.input_size,
                                                x.device, self.storage_dtype)
        archive = self.archive
        if x.dtype == torch.bfloat16 and self.dense_retrieval:
            archive.keep_bf16_copy()
        # the carried state stays fp32 whatever the activations are
        memory = c_init.float() if c_init is not None else torch.zeros(B, self.hidden, self.key_dim,
                                                                       device=x.device, dtype=torch.float32)
        # Everything that depends on the layer input alone is computed for the whole sequence at once
        # (paper_grm.py:491-493, 522-523, 566-570 do it segment by segment): the three projections of
        # the memory cell, the routing queries and the segment summaries.  Only the scan, the routing
        # against the archive and the retrieval are sequential in the segments.

        def per_segment(t: Tensor) -> List[Tensor]:
            if segment_major:
                return list(t.unbind(0))
            return [t[:, s0:s1].contiguous() for s0, s1 in bounds]

        k_all, q_all = self._keys_and_queries(x)
        k_seg = per_segment(k_all)
        v_seg = per_segment(_linear(x, self.p, "memory_cell.value_proj"))
        q_seg = per_segment(q_all)
        # summaries [B, n, D]: mean of the fp32 input over each segment (paper_grm.py:522-523)
        if segment_major:
            summaries = x.mean(dim=2, dtype=torch.float32).transpose(0, 1)
        elif bounds:
            summaries = torch.stack([x[:, s0:s1].mean(dim=1, dtype=torch.float32) for s0, s1 in bounds], dim=1)
        else:
            summaries = x.new_zeros(B, 0, x.shape[-1], dtype=torch.float32)
        summaries = archive.as_stored(summaries)
        summary_seg = [summaries[:, i] for i in range(len(bounds))]
        # The routing keys of this call's segments are projected once, here, and archived with them
        # (the reference projects the archived summaries again in every segment, paper_grm.py:566-570;
        # the weights do not change during a forward pass).  The queries are only needed if some
        # segment will see a non-empty archive.
        route_q_weight = self._fp32_param("gating_unit.query_projection.weight")
        self._route_key_weight = self._fp32_param("gating_unit.key_projection.weight")
        fold = self.fold_routing_projection and self.input_size <= 2 * self.route_dim
        self._route_query_weight = route_q_weight if fold else None
        route_key_all = self._route_keys(summaries)
        route_key_seg = [route_key_all[:, i] for i in range(len(bounds))]
        if archive.count > 0 and archive.route_keys is None:       # an archive restored from a saved state
            archive.set_route_keys(self._route_keys(archive.ordered_summaries()))
        if archive.write_ahead(summaries, route_key_all):
            summary_seg = [None] * len(bounds)
        if archive.count > 0 or len(bounds) > 1:
            # folded, the router scores the layer input itself; bf16 input is read as it is (widening is
            # exact, so the scores are those of the fp32 copy)
            rq_seg = per_segment(x if fold else F.linear(x.float(), route_q_weight))

        hidden_seg: List[Tensor] = []
        routes = []
        for i in range(len(bounds)):
            h_online, memory = cuda_ops.cuda_chunk_update(k_seg[i], v_seg[i], q_seg[i], memory, self.decay)
            if archive.count > 0:                                   # paper_grm.py:620-621: no fusion otherwise
                if archive.head == 0 and archive.capacity <= 16:
                    # the whole ring with the number of archived segments as the visible count: the
                    # same selection as over ring[:, :count], without copying that slice
                    gates, indices = self._route(rq_seg[i], archive.route_keys,
                                                 self._visible_counts(rq_seg[i].shape[1], archive.count, x.device))
                else:
                    gates, indices = self._route(rq_seg[i], archive.ordered_route_keys())
                h = self._retrieve_and_fuse(q_seg[i], h_online, gates, indices)
                if return_routes:
                    routes.append((gates, indices))
            else:
                h = h_online
            hidden_seg.append(h)
            archive.push(memory, summary_seg[i], route_key_seg[i])  # paper_grm.py:522-523, 721-725
            if self.init_mode == "independent":
                memory = torch.zeros_like(memory)
        if hidden_seg:
            last_hidden = hidden_seg[-1][:, -1]
            hidden = torch.stack(hidden_seg, dim=0) if segment_major else torch.cat(hidden_seg, dim=1)
            out = _linear(hidden, self.p, "output_proj")
        else:
            last_hidden = torch.zeros(B, self.hidden, device=x.device, dtype=x.dtype)
            out = x.new_zeros(B, 0, self.p["output_proj.weight"].shape[0])
        aux = {"num_segments": archive.count, "total_pushed": archive.total_pushed}
        if return_routes:
            aux["routes"] = routes
        return out, last_hidden, memory, aux


class StackedSegmentMemoryRunner:
    """``HierarchicalSegmentMemoryModel`` (grm/core/multilayer_grm.py:105-220), optionally under the
    language-model wrapper (embedding + vocabulary projection, grm/utils/train.py:192-225).

    ``params`` uses the reference names: ``layers.<i>.grm.<...>``, ``layers.<i>.layer_norm.*``,
    ``output_proj.*`` and, for the language model, ``embedding.weight`` / ``output_layer.*`` with the
    stack under ``grm_rnn.``.
    """

    def __init__(self, params: Dict[str, Tensor], num_layers: int, *, language_model: bool = False, **layer_kwargs):
        prefix = "grm_rnn." if language_model else ""
        self.language_model = language_model
        self.params = params
        self.prefix = prefix
        self.layers = []
        for i in range(num_layers):
            base = f"{prefix}layers.{i}.grm."
            sub = {k[len(base):]: v for k, v in params.items() if k.startswith(base)}
            self.layers.append(SegmentMemoryRunner(sub, **layer_kwargs))
        self.num_layers = num_layers
        # False: stop after the stack's own output projection (the 512 -> vocabulary layer of the language-model
        # wrapper is not part of the memory path; timing with and without it separates the two)
        self.vocabulary_projection = True
        self._fp32_cache: Dict[int, Tuple[Tensor, Tensor, int]] = {}

    def _add_layer_norm(self, out: Tensor, h: Tensor, weight: Optional[Tensor], bias: Optional[Tensor]) -> Tensor:
        """``LayerNorm(out + h)`` in one pass (``torch.ops.grmx.add_layer_norm``: sum and normalisation in fp32,
        no rounded intermediate; multilayer_grm.py:93,96)."""
        H = h.shape[-1]
        per16 = 4 if h.dtype == torch.float32 else 8
        if not (h.is_cuda and h.dtype == out.dtype and h.dtype in (torch.float32, torch.bfloat16) and H <= 1024
                and H % per16 == 0 and weight is not None and bias is not None):
            return F.layer_norm(out + h, (H,), weight, bias, 1e-5)
        params = []
        for t in (weight, bias):
            cached = self._fp32_cache.get(id(t))
            if cached is None or cached[0] is not t or cached[2] != t._version:
                cached = (t, t.float(), t._version)
                self._fp32_cache[id(t)] = cached
            params.append(cached[1])
        return torch.ops.grmx.add_layer_norm(h, out, params[0], params[1], 1e-5)

    @torch.no_grad()
    def forward(self, x: Tensor, reset_memory: bool = True):
        p, pre = self.params, self.prefix
        B, T = x.shape[0], x.shape[1]
        lengths = {layer.segment_length for layer in self.layers}
        L = next(iter(lengths))
        # whole segments of one length in every layer: keep segment i of all batch rows contiguous from
        # the embedding to the last layer, so that no layer transposes its input or its output
        act_dtype = p["embedding.weight"].dtype if self.language_model else x.dtype
        probe = torch.empty(B, T, 0, device=x.device, dtype=act_dtype)
        whole = all(layer.whole_sequence_applies(probe, reset_memory) for layer in self.layers)
        segment_major = len(lengths) == 1 and T > 0 and T % L == 0 and not whole
        if segment_major:
            x = x.reshape(B, T // L, L, *x.shape[2:]).transpose(0, 1).contiguous()
        h = F.embedding(x, p["embedding.weight"]) if self.language_model else x
        finals = []
        for i, layer in enumerate(self.layers):
            if segment_major:
                out, _, memory, _ = layer.forward_segment_major(h, reset_memory=reset_memory)
            else:
                out, _, memory, _ = layer.forward(h, reset_memory=reset_memory)
            w, b = p.get(f"{pre}layers.{i}.layer_norm.weight"), p.get(f"{pre}layers.{i}.layer_norm.bias")
            h = self._add_layer_norm(out, h, w, b)                      # multilayer_grm.py:88-92
            finals.append(memory)
        if segment_major:
            h = h.transpose(0, 1).reshape(B, T, h.shape[-1])
        y = F.linear(h, p[f"{pre}output_proj.weight"], p.get(f"{pre}output_proj.bias"))
        if self.language_model and self.vocabulary_projection:
            y = F.linear(y, p["output_layer.weight"], p.get("output_layer.bias"))
        _check_errors_if_asked()
        return y, torch.stack(finals, dim=0)


class GraphedForward:
    """A runner's forward pass for one input shape, captured once as a CUDA graph and replayed.

    A forward pass is hundreds of small launches per layer (projections, normalisations, the kernels
    of this package, one set per segment), and the segment loop is static for a given sequence length
    when the archive is reset at the start of the call: the number of archived segments every
    segment sees is known in advance.  Replaying the captured graph removes the host from the loop.
    The inputs are copied into the buffer the graph was captured on; the outputs are the graph's own
    buffers and are overwritten by the next call.
    """

    def __init__(self, runner, example_input: Tensor, warmup: int = 2):
        if example_input.device.type != "cuda":
            raise RuntimeError("GraphedForward needs a CUDA tensor")
        self._input = example_input.clone()
        side = torch.cuda.Stream(device=example_input.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):                       # first calls set kernel attributes, fill caches
                runner.forward(self._input, reset_memory=True)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._output = runner.forward(self._input, reset_memory=True)

    def __call__(self, x: Tensor):
        self._input.copy_(x)
        self._graph.replay()
        return self._output


def language_model_parameter_shapes(num_layers: int, hidden: int, key_dim: int, vocab: int, embed_dim: int,
                                    route_dim: Optional[int] = None) -> Dict[str, Tuple[int, ...]]:
    """Names and shapes of the parameters ``StackedSegmentMemoryRunner(language_model=True)`` reads, as
    the reference's ``SegmentMemoryLanguageModel.state_dict()`` lays them out (grm/utils/train.py:192-225,
    grm/core/multilayer_grm.py:105-160, grm/core/paper_grm.py:405-470).  Layer 0 takes the embedding,
    the others the hidden state; the routing dimension defaults to the hidden size."""
    route_dim = hidden if route_dim is None else route_dim
    shapes: Dict[str, Tuple[int, ...]] = {"embedding.weight": (vocab, embed_dim)}
    for i in range(num_layers):
        d_in = embed_dim if i == 0 else hidden
        base = f"grm_rnn.layers.{i}.grm."
        shapes.update({
            base + "memory_cell.key_proj.weight": (key_dim, d_in), base + "memory_cell.key_proj.bias": (key_dim,),
            base + "memory_cell.value_proj.weight": (hidden, d_in), base + "memory_cell.value_proj.bias": (hidden,),
            base + "memory_cell.query_proj.weight": (key_dim, d_in), base + "memory_cell.query_proj.bias": (key_dim,),
            base + "gating_unit.query_projection.weight": (route_dim, d_in),
            base + "gating_unit.key_projection.weight": (route_dim, d_in),
            base + "aggregator.layer_norm.weight": (hidden,), base + "aggregator.layer_norm.bias": (hidden,),
            base + "output_proj.weight": (hidden, hidden), base + "output_proj.bias": (hidden,),
            f"grm_rnn.layers.{i}.layer_norm.weight": (hidden,), f"grm_rnn.layers.{i}.layer_norm.bias": (hidden,),
        })
    shapes.update({"grm_rnn.output_proj.weight": (hidden, hidden), "grm_rnn.output_proj.bias": (hidden,),
                   "output_layer.weight": (vocab, hidden), "output_layer.bias": (vocab,)})
    return shapes

