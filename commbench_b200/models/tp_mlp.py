"""Tensor-parallel MLP block built from the fused kernels (the flagship step of ``bench.py``).

Sequence-parallel in, sequence-parallel out (Megatron "SP + TP" layout):

    x_local [T/W, H]  --AG->GEMM-->  h [T, I/W]  --GEMM->RS-->  y_local [T/W, H]

with ``W1`` column-sharded ``[I/W, H]`` and ``W2`` row-sharded ``[H, I/W]``.  The shapes of
the headline configuration (T=8192 tokens, H=8192, I=28672) are the ones the reference's
fused examples sweep towards (datasets/example051_thunderkitten_ag_gemm_easy/nv/
empty_thunderkitten_ag_gemm.cu:539-543 and datasets/example054_thunderkitten_gemm_rs_easy/nv/
empty_thunderkitten_gemm_rs.cu:514), which stop at one GEMM each; chaining the two gives a
complete transformer MLP without any standalone collective.

``forward``          fused path (2 kernel launches of this library; 2 plain tcgen05 GEMMs at W=1)
``forward_unfused``  the baseline: NCCL all-gather + cuBLAS matmul + cuBLAS matmul + NCCL
                     reduce-scatter on the same tensors
``forward_host``     end-to-end call: pinned host tokens in, scalar metric out
"""
from __future__ import annotations

import torch

from ..ops.gemm import gemm
from ..ops.tp import AgGemm, GemmRs, stream_write_u32
from ..ops.util import abs_mean


class TPMLP:
    def __init__(self, ctx, hidden: int, intermediate: int, max_tokens: int, seed: int = 0,
                 activation: str | None = None, gate_host_copy: bool = False):
        self.ctx = ctx
        self.world = ctx.world
        self.rank = ctx.rank
        self.hidden, self.intermediate, self.max_tokens = hidden, intermediate, max_tokens
        if intermediate % self.world or max_tokens % (128 * self.world):
            raise ValueError("intermediate must divide by world and tokens by 128*world")
        self.i_local = intermediate // self.world
        dev = ctx.device
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + self.rank)
        # random-init weights N(0, 0.02): this rank's shards only
        self.w1 = (torch.randn(self.i_local, hidden, device=dev, generator=g) * 0.02).bfloat16()
        self.w2 = (torch.randn(hidden, self.i_local, device=dev, generator=g) * 0.02).bfloat16()
        self.activation = activation
        # End-to-end path: launch AG->GEMM while the tokens are still being copied from the host
        # and let it consume rows as they land (see _forward_host_gated).  Measured on 1, 2 and 4
        # B200s it ends level with the simpler schedule (the block run on two row halves, the
        # second half's copy under the first half's kernels), so it is opt-in.
        self.gate_host_copy = gate_host_copy
        if self.world > 1 or gate_host_copy:
            self.ag = AgGemm(ctx, max_m=max_tokens, k=hidden)
        if self.world > 1:
            self.rs = GemmRs(ctx, max_m=max_tokens, max_n=hidden)
        self.h = torch.empty(max_tokens, self.i_local, dtype=torch.bfloat16, device=dev)
        self.y = torch.empty(max_tokens // self.world, hidden, dtype=torch.bfloat16, device=dev)
        self._x_dev = torch.empty(max_tokens // self.world, hidden, dtype=torch.bfloat16, device=dev)
        self._metric_host = torch.empty(1, dtype=torch.float32).pin_memory() \
            if torch.cuda.is_available() else torch.empty(1)
        self.launches_per_step = 2
        self._copy_stream = None
        self._copy_events = None
        self._ready = None          # per-256-row "has landed" words of the gated end-to-end path
        self._ready_seq = 0

    # ---------------------------------------------------------------- fused path
    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        T = x_local.shape[0] * self.world
        h = self.h[:T]
        y = self.y[:x_local.shape[0]]
        if self.world == 1:
            gemm(x_local, self.w1, out=h)
            if self.activation == "silu":
                torch.nn.functional.silu(h, inplace=True)
            gemm(h, self.w2, out=y)
            return y
        self.ag(x_local, self.w1, out=h)
        if self.activation == "silu":
            torch.nn.functional.silu(h, inplace=True)
        self.rs(h, self.w2, out=y)
        return y

    # ------------------------------------------------------------ unfused baseline
    def forward_unfused(self, x_local: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        if self.world == 1:
            h = torch.matmul(x_local, self.w1.t())
            if self.activation == "silu":
                torch.nn.functional.silu(h, inplace=True)
            return torch.matmul(h, self.w2.t())
        x_full = torch.empty(x_local.shape[0] * self.world, self.hidden, dtype=x_local.dtype,
                             device=x_local.device)
        dist.all_gather_into_tensor(x_full, x_local)
        h = torch.matmul(x_full, self.w1.t())
        if self.activation == "silu":
            torch.nn.functional.silu(h, inplace=True)
        part = torch.matmul(h, self.w2.t())
        y = torch.empty(x_local.shape[0], self.hidden, dtype=x_local.dtype, device=x_local.device)
        dist.reduce_scatter_tensor(y, part)
        return y

    # ---------------------------------------------------------------- end to end
    def _rows_forward(self, x_rows: torch.Tensor, h: torch.Tensor, y: torch.Tensor, fused: bool):
        """The whole block on a group of local rows (W > 1): y = MLP(x_rows), with the gathered
        intermediate in ``h`` ([W * rows, I/W])."""
        import torch.distributed as dist

        if fused:
            self.ag(x_rows, self.w1, out=h)
            if self.activation == "silu":
                torch.nn.functional.silu(h, inplace=True)
            self.rs(h, self.w2, out=y)
            return
        x_full = torch.empty(x_rows.shape[0] * self.world, self.hidden, dtype=x_rows.dtype,
                             device=x_rows.device)
        dist.all_gather_into_tensor(x_full, x_rows)
        torch.matmul(x_full, self.w1.t(), out=h)
        if self.activation == "silu":
            torch.nn.functional.silu(h, inplace=True)
        dist.reduce_scatter_tensor(y, torch.matmul(h, self.w2.t()))

    def _forward_host_pipelined(self, x_host_pinned: torch.Tensor, chunks: int,
                                fused: bool) -> torch.Tensor:
        """The host-to-device copy of the tokens is cut into row chunks on a copy stream and the
        work on chunk i runs while chunk i+1 is still on the wire.  One rank: the first GEMM runs
        per chunk, the second once over all rows.  Several ranks: the whole block runs per chunk
        (chunk c of every rank is gathered, multiplied, reduced and scattered back: exactly
        y[c] = MLP(x[c]) for every rank).  The same schedule serves the fused kernels and the
        unfused NCCL + cuBLAS composition."""
        n = x_host_pinned.shape[0]
        rows = n // chunks
        W = self.world
        main = torch.cuda.current_stream()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream()
            self._copy_events = [torch.cuda.Event() for _ in range(16)]
        cs = self._copy_stream
        cs.wait_stream(main)           # the previous step's readers of the staging buffer are done
        xd = self._x_dev[:n]
        with torch.cuda.stream(cs):
            for c in range(chunks):
                xd[c * rows:(c + 1) * rows].copy_(x_host_pinned[c * rows:(c + 1) * rows],
                                                  non_blocking=True)
                self._copy_events[c].record(cs)
        h = self.h[:n * W]
        y = self.y[:n]
        for c in range(chunks):
            main.wait_event(self._copy_events[c])
            xc = xd[c * rows:(c + 1) * rows]
            if W == 1:
                if fused:
                    gemm(xc, self.w1, out=h[c * rows:(c + 1) * rows])
                else:
                    torch.matmul(xc, self.w1.t(), out=h[c * rows:(c + 1) * rows])
            else:
                self._rows_forward(xc, h[c * rows * W:(c + 1) * rows * W],
                                   y[c * rows:(c + 1) * rows], fused)
        if W == 1:
            if self.activation == "silu":
                torch.nn.functional.silu(h, inplace=True)
            if fused:
                gemm(h, self.w2, out=y)
            else:
                torch.matmul(h, self.w2.t(), out=y)
        return y

    GATE_ROWS = 256

    def _forward_host_gated(self, x_host_pinned: torch.Tensor) -> torch.Tensor:
        """Fused path: the AG->GEMM kernel is launched at once and consumes the
        local rows as the host-to-device copy delivers them.  The copy runs on its own stream in
        pieces of 256 rows or more (16 pieces at most), each followed by a stream memory operation
        that publishes "these rows have landed"; the kernel's communication CTAs push, and its
        tensor-core CTAs multiply, a row block as soon as its word is set.  One launch per GEMM,
        whatever the piece count.  The kernels are enqueued BEFORE the copies, so the host's time
        to enqueue the pieces overlaps the first pieces' transfer."""
        n = x_host_pinned.shape[0]
        g = self.GATE_ROWS
        while n // g > 16 and n % (2 * g) == 0:
            g *= 2
        main = torch.cuda.current_stream()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream()
            self._copy_events = [torch.cuda.Event() for _ in range(16)]
        if self._ready is None:
            self._ready = torch.zeros(self.max_tokens // self.world // self.GATE_ROWS + 1,
                                      dtype=torch.int32, device=self._x_dev.device)
            torch.cuda.synchronize(self._x_dev.device)
        cs = self._copy_stream
        # The previous step's kernels are done with the staging rows before they are overwritten;
        # the copy stream must NOT wait for the kernels enqueued below, which wait for it.
        self._copy_events[0].record(main)
        cs.wait_event(self._copy_events[0])
        self._ready_seq += 1
        xd = self._x_dev[:n]
        h = self.h[:n * self.world]
        y = self.y[:n]
        self.ag(xd, self.w1, out=h, src_ready=(self._ready, self._ready_seq, g))
        if self.activation == "silu":
            torch.nn.functional.silu(h, inplace=True)
        if self.world == 1:
            gemm(h, self.w2, out=y)
        else:
            self.rs(h, self.w2, out=y)
        with torch.cuda.stream(cs):
            for c in range(n // g):
                xd[c * g:(c + 1) * g].copy_(x_host_pinned[c * g:(c + 1) * g], non_blocking=True)
                stream_write_u32(self._ready[c:c + 1], self._ready_seq, cs)
        return y

    def host_chunks(self, n_local: int) -> int:
        """Row chunks of the pipelined end-to-end path.  One rank: four (only the first GEMM is
        cut).  Several ranks: two, as long as every launch keeps 4096 gathered rows and 1024
        local rows - smaller launches lose more to partly filled tile waves than the overlap
        of the copy gains."""
        if self.world == 1:
            return 4 if n_local % 1024 == 0 and n_local >= 8192 else 1
        if n_local % 512 == 0 and n_local // 2 >= 1024 and (n_local // 2) * self.world >= 4096:
            return 2
        return 1

    def forward_host(self, x_host_pinned: torch.Tensor, fused: bool = True) -> float:
        """Tokens arrive in pinned host memory; returns mean(|y|) read back to the host."""
        n = x_host_pinned.shape[0]
        chunks = self.host_chunks(n)
        if fused and self.gate_host_copy and n % self.GATE_ROWS == 0 and n >= 2 * self.GATE_ROWS:
            y = self._forward_host_gated(x_host_pinned)
        elif chunks > 1:
            y = self._forward_host_pipelined(x_host_pinned, chunks, fused)
        else:
            xd = self._x_dev[:n]
            xd.copy_(x_host_pinned, non_blocking=True)
            y = self.forward(xd) if fused else self.forward_unfused(xd)
        m = abs_mean(y)                 # one pass over y, one launch
        self._metric_host.copy_(m, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(self._metric_host[0])

    def flops(self, tokens: int) -> float:
        """FLOPs of one step over the WHOLE job (all ranks)."""
        return 2.0 * 2.0 * tokens * self.hidden * self.intermediate
