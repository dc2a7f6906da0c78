"""The scale-out form of the memory path: many independent (batch, head) rows, sharded over the GPUs of
one box, streamed through each GPU in slabs.

Every row is a scan of its own with an archive of its own (the reference indexes the archive within a
batch row, grm/csrc/batched_gather.cu:38-41, and drives one chunk update per segment,
grm/core/paper_grm.py:702-728), so rank ``r`` of ``world`` takes the contiguous rows
``sharding.row_range(rows, r, world)`` and nothing crosses GPUs on the data path.  A rank's rows do not
fit its memory at once at the full shape (4096 rows x 32768 tokens x 128 features: 34 GB per tensor), so
they go through in slabs of ``slab_rows`` rows whose inputs are generated on the device.

Per slab: one scan launch over all segments that leaves every segment-end state in the slab's archive
(``grmx_chunk_scan_fwd_segments``), segment-level routing (query = mean of the segment's q, key = mean of
its k, causal top-k) and the fused retrieval from that archive (``grmx_retrieve_fuse``, residual +
LayerNorm).

Verification rows: a few rows per rank take inputs generated on the host from the row's own seed
(``host_row_inputs``), so that anyone can regenerate exactly those rows later and check the outputs the
GPU produced for them; they sit in the same slab and the same launches as their neighbours.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Tuple

from .sharding import row_range


@dataclass(frozen=True)
class ScaleOutShape:
    rows: int = 4096          # batch 256 x 16 heads
    heads: int = 16
    tokens: int = 32768
    dim: int = 128            # d_k = d_v
    segment: int = 1024
    top_k: int = 8
    decay: float = 0.97

    @property
    def segments(self) -> int:
        return self.tokens // self.segment

    @property
    def batch_tokens(self) -> int:
        """Tokens as the metric counts them: batch x sequence (heads are not extra tokens)."""
        return self.rows // self.heads * self.tokens

    def scan_bytes_per_row(self) -> int:
        """Algorithmic bytes of the scan for one row: q, k, v in and the hidden states out, bf16."""
        return self.tokens * (2 * (2 * self.dim + self.dim) + 2 * self.dim)


def plan_slabs(shape: ScaleOutShape, rank: int, world: int, slab_rows: int) -> List[Tuple[int, int]]:
    """Half-open global row intervals this rank processes, one per slab, in order."""
    if slab_rows <= 0:
        raise ValueError("slab_rows must be positive")
    start, stop = row_range(shape.rows, rank, world)
    return [(r0, min(r0 + slab_rows, stop)) for r0 in range(start, stop, slab_rows)]


def sample_rows(shape: ScaleOutShape, rank: int, world: int, per_rank: int) -> List[int]:
    """Global indices of the verification rows of this rank: spread evenly over its rows, first and last
    included when there are two or more."""
    start, stop = row_range(shape.rows, rank, world)
    n = min(per_rank, stop - start)
    if n <= 0:
        return []
    if n == 1:
        return [start]
    return sorted({start + round(i * (stop - 1 - start) / (n - 1)) for i in range(n)})


def host_row_inputs(shape: ScaleOutShape, row: int, seed: int = 0):
    """Inputs of one verification row from its own seed, on the host: ``(q, k, v, online)`` as bf16 /
    fp32 torch tensors -- q, k ~ N(0,1) L2-normalised, v ~ N(0,1), the online state the retrieval is fused
    with ~ N(0,1) per segment."""
    import torch

    g = torch.Generator().manual_seed(seed * 1_000_003 + row)
    T, d = shape.tokens, shape.dim
    q = torch.nn.functional.normalize(torch.randn(T, d, generator=g), dim=-1, eps=1e-6)
    k = torch.nn.functional.normalize(torch.randn(T, d, generator=g), dim=-1, eps=1e-6)
    v = torch.randn(T, d, generator=g)
    online = torch.randn(shape.segments, d, generator=g)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16), online


class SlabRunner:
    """Device buffers of one slab and the launches that process it (CUDA only)."""

    def __init__(self, shape: ScaleOutShape, slab_rows: int, device):
        import torch

        from . import cabi

        self.shape, self.rows, self.device = shape, slab_rows, device
        self.lib = cabi.load()
        self.cabi = cabi
        R, T, d, S = slab_rows, shape.tokens, shape.dim, shape.segments
        bf = dict(device=device, dtype=torch.bfloat16)
        self.q, self.k, self.v = (torch.empty(R, T, d, **bf) for _ in range(3))
        self.hidden = torch.empty(R, T, d, **bf)
        self.m_in = torch.zeros(R, d, d, device=device)
        self.m_out = torch.empty(R, d, d, device=device)
        self.archive = torch.empty(R, S, d, d, device=device)
        self.online = torch.empty(R, S, d, device=device)
        self.seg_q = torch.empty(R, S, d, device=device)
        self.seg_k = torch.empty(R, S, d, device=device)
        self.visible = torch.arange(S, device=device, dtype=torch.int32)
        self.indices = torch.empty(R, S, shape.top_k, device=device, dtype=torch.int64)
        self.gates = torch.empty(R, S, shape.top_k, device=device)
        self.fused = torch.empty(R, S, d, device=device)

    def bytes_held(self) -> int:
        tensors = (self.q, self.k, self.v, self.hidden, self.m_in, self.m_out, self.archive, self.online, self.seg_q,
                   self.seg_k, self.indices, self.gates, self.fused)
        return sum(t.numel() * t.element_size() for t in tensors)

    def generate(self, r0: int, r1: int, seed: int, host_rows: Dict[int, tuple]) -> int:
        """Fill the inputs of rows [r0, r1) on the device (one generator per slab, seeded by the slab's
        first row), then overwrite the verification rows among them with their host-generated inputs.
        Generated a few rows at a time, so that the fp32 temporaries stay small."""
        import torch

        n = r1 - r0
        g = torch.Generator(device=self.device).manual_seed(seed * 1_000_003 + 7919 * (r0 + 1))
        T, d = self.shape.tokens, self.shape.dim
        step = 32
        for a in range(0, n, step):
            b = min(a + step, n)
            for dst, unit in ((self.q, True), (self.k, True), (self.v, False)):
                t = torch.randn(b - a, T, d, device=self.device, generator=g)
                if unit:
                    t = torch.nn.functional.normalize(t, dim=-1, eps=1e-6)
                dst[a:b].copy_(t)
        self.online[:n].copy_(torch.randn(n, self.shape.segments, d, device=self.device, generator=g))
        for row, (q, k, v, online) in host_rows.items():
            if r0 <= row < r1:
                i = row - r0
                self.q[i].copy_(q)
                self.k[i].copy_(k)
                self.v[i].copy_(v)
                self.online[i].copy_(online)
        return n

    def segment_means(self, n: int) -> None:
        """Routing queries and keys of the slab: per-segment means of q and k in fp32 (input preparation,
        the reference forms its segment summaries the same way, grm/core/paper_grm.py:522-523)."""
        import torch

        S, L, d = self.shape.segments, self.shape.segment, self.shape.dim
        torch.mean(self.q[:n].view(n, S, L, d), dim=2, dtype=torch.float32, out=self.seg_q[:n])
        torch.mean(self.k[:n].view(n, S, L, d), dim=2, dtype=torch.float32, out=self.seg_k[:n])

    def launch(self, n: int, stream: int, after_scan=None) -> int:
        """Scan with segment snapshots -> routing -> fused retrieval for the first ``n`` rows; returns the
        number of kernel launches enqueued.  ``after_scan`` is called between the scan and the retrieval
        (the benchmark records an event there)."""
        sh, lib, cabi = self.shape, self.lib, self.cabi
        before = lib.grmx_launch_count()
        cabi.check(lib.grmx_chunk_scan_fwd_segments(
            self.k.data_ptr(), self.v.data_ptr(), self.q.data_ptr(), self.m_in.data_ptr(), self.hidden.data_ptr(),
            self.m_out.data_ptr(), self.archive.data_ptr(), sh.segments, 0, sh.segment, n, sh.tokens, sh.dim, sh.dim,
            sh.decay, cabi.BF16, cabi.F32, stream))
        if after_scan is not None:
            after_scan()
        cabi.check(lib.grmx_topk_route(self.seg_q.data_ptr(), self.seg_k.data_ptr(), self.visible.data_ptr(), n,
                                       sh.segments, sh.segments, sh.dim, sh.top_k, 1.0, 1.0, self.indices.data_ptr(),
                                       self.gates.data_ptr(), None, stream))
        cabi.check(lib.grmx_retrieve_fuse(self.archive.data_ptr(), self.indices.data_ptr(), self.gates.data_ptr(),
                                          self.seg_q.data_ptr(), self.online.data_ptr(), None, None, 1e-5,
                                          self.fused.data_ptr(), n, sh.segments, sh.segments, sh.top_k, sh.dim, sh.dim,
                                          cabi.FUSE_RESIDUAL_LN, stream))
        return int(lib.grmx_launch_count() - before)


def scale_out_bytes(shape: ScaleOutShape, rows: int) -> int:
    """Algorithmic bytes of the whole path for ``rows`` rows: the scan's tokens in and out, the archive
    written once (fp32) and read by the retrieval (top_k matrices per segment query, fewer while fewer
    are visible)."""
    d, S = shape.dim, shape.segments
    routed = sum(min(shape.top_k, j) for j in range(S))
    return rows * (shape.scan_bytes_per_row() + S * d * d * 4 + routed * d * d * 4)


def pack_sample(hidden_row, m_out_row, fused_row, indices_row):
    """One verification row's outputs as a flat fp32 vector (for a single gather): hidden states
    [T, d] (bf16 values), final memory [d, d], fused retrieval [S, d], routing indices [S, top_k]."""
    import torch

    return torch.cat([hidden_row.float().flatten(), m_out_row.flatten(), fused_row.flatten(),
                      indices_row.float().flatten()])


def unpack_sample(flat, shape: ScaleOutShape):
    T, d, S, R = shape.tokens, shape.dim, shape.segments, shape.top_k
    sizes = [T * d, d * d, S * d, S * R]
    parts, at = [], 0
    for n in sizes:
        parts.append(flat[at:at + n])
        at += n
    return parts[0].view(T, d), parts[1].view(d, d), parts[2].view(S, d), parts[3].view(S, R).round().long()


def sample_vector_len(shape: ScaleOutShape) -> int:
    return shape.tokens * shape.dim + shape.dim * shape.dim + shape.segments * shape.dim + shape.segments * shape.top_k


def n_slabs_for(shape: ScaleOutShape, world: int, slab_rows: int) -> int:
    return max(len(plan_slabs(shape, r, world, slab_rows)) for r in range(world))


def per_gpu_hbm_fraction(shape: ScaleOutShape, rows_done: int, seconds: float, hbm_gbs: float) -> float:
    if seconds <= 0:
        return math.nan
    return rows_done * shape.scan_bytes_per_row() / seconds / 1e9 / hbm_gbs
