"""The W4A16 feed-forward chain: ``down( silu(x @ W_gate) * (x @ W_up) )``.

Three launches per rank: one W4A16 GEMM over the concatenated gate|up weights (f16 out,
``[M, 2*I]``), the SiLU-gate pass over its two halves, and the W4A16 down projection (f32 out).
KAIO has the pieces (``matmul_int4``, kaio-ops/src/matmul_int4_kernel.rs:2126-2171; the
``fused_silu_gate`` user kernel, examples/fused_silu_gate/src/main.rs:13-21) but no chain and no
multi-device form; this is the caller one level above the quantized GEMMs.

Across ``P`` ranks the chain is column-parallel then row-parallel: rank ``r`` owns columns
``[r*I/P, (r+1)*I/P)`` of W_gate and W_up and the matching K-rows of W_down, so the intermediate
never leaves the GPU (no all-gather of ``[M, I]``) and the only exchange is the sum of the
``[M, H]`` f32 partial outputs: an all-reduce, or a reduce-scatter when each rank only needs its
own ``M/P`` rows.  With ``reduce="fused"`` the sum does not go through NCCL: the down projection's
epilogue stores its partial tiles straight into staging slots of the other ranks (peer memory,
symmetric allocation), the ranks meet at a barrier, and a small kernel adds the slots in rank order
(bit-identical on every rank and run).  Small outputs go whole to every rank (one step, one
barrier); large ones are scattered by column block and the summed blocks are stored back to every
rank (two steps, the traffic of a ring all-reduce).

For large M (``reduce="overlap"``, :meth:`FfnInt4.run_overlapped`) the NCCL all-reduce is hidden
behind the GEMMs: the weights are dequantised once per call, the rows are cut into a few chunks, and
chunk ``i``'s partial rows are summed on a second stream while chunk ``i+1`` is computed.

The helpers at the top are layout logic and run on CPU tensors too.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .sharding import shard_bounds, shard_group_scales, shard_packed_int4

GROUP = 128


def k_shard_bounds(k: int, world: int, rank: int) -> tuple[int, int]:
    """K range of ``rank`` for a row-parallel W4A16 GEMM: equal shards, each a whole number of
    128-wide scale groups."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if k % (world * GROUP) != 0:
        raise ValueError(f"K={k} does not split into {world} shards of whole {GROUP}-wide groups")
    w = k // world
    return rank * w, (rank + 1) * w


def k_shard_packed_int4(packed: torch.Tensor, k: int, n: int, world: int, rank: int) -> torch.Tensor:
    """Packed s4 weights keep the K words of a column contiguous (word ``k/8`` of column ``j`` at
    ``(k/8) + j*(K/8)``), so a K range is a strided slice of every column: copied once into a
    packed ``[N][K/P/8]`` buffer of the same layout."""
    lo, hi = k_shard_bounds(k, world, rank)
    return packed.view(-1)[: n * (k // 8)].view(n, k // 8)[:, lo // 8:hi // 8].contiguous().view(-1)


def k_shard_group_scales(scales: torch.Tensor, k: int, n: int, world: int, rank: int) -> torch.Tensor:
    """f16 ``[K/128, N]`` group scales: a K range is a contiguous range of rows (a view)."""
    lo, hi = k_shard_bounds(k, world, rank)
    return scales.view(-1)[: (k // GROUP) * n].view(k // GROUP, n)[lo // GROUP:hi // GROUP].reshape(-1)


def concat_gate_up(w_gate: torch.Tensor, s_gate: torch.Tensor, w_up: torch.Tensor, s_up: torch.Tensor,
                   k: int, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Gate and up projections as ONE ``[K, 2N]`` W4A16 weight: packed columns are contiguous, so
    the packed buffers concatenate flat; the scales concatenate along their column axis."""
    packed = torch.cat([w_gate.view(-1)[: n * (k // 8)], w_up.view(-1)[: n * (k // 8)]])
    g = k // GROUP
    scales = torch.cat([s_gate.view(-1)[: g * n].view(g, n), s_up.view(-1)[: g * n].view(g, n)], dim=1)
    return packed, scales.contiguous().view(-1)


def interleave_index(n: int, block: int = 64) -> torch.Tensor:
    """Column order of the fused gate|up + SiLU-gate GEMM: position ``p`` of the interleaved
    ``[K, 2n]`` weight takes column ``index[p]`` of the concatenated ``[gate | up]`` weight -- blocks
    of ``block`` gate columns alternate with the same columns of up."""
    if n % block != 0:
        raise ValueError(f"n={n} must be a multiple of the interleave block {block}")
    p = torch.arange(2 * n)
    b, within = p // (2 * block), p % (2 * block)
    return torch.where(within < block, b * block + within, n + b * block + within - block)


def interleave_gate_up(w_gu: torch.Tensor, s_gu: torch.Tensor, k: int, n: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The concatenated ``[K, 2n]`` gate|up weight of :func:`concat_gate_up` re-ordered for
    ``matmul_int4_silu_gate`` (packed columns are contiguous runs of ``K/8`` words; scales are
    ``[K/128, 2n]``)."""
    idx = interleave_index(n).to(w_gu.device)
    packed = w_gu.view(-1)[: 2 * n * (k // 8)].view(2 * n, k // 8)[idx].contiguous().view(-1)
    g = k // GROUP
    scales = s_gu.view(-1)[: g * 2 * n].view(g, 2 * n)[:, idx].contiguous().view(-1)
    return packed, scales


class FfnInt4:
    """One rank's share of the W4A16 feed-forward block.

    ``w_gate``/``w_up`` are packed ``[hidden, inter]`` weights with ``[hidden/128, inter]`` f16
    scales; ``w_down`` is packed ``[inter, hidden]`` with ``[inter/128, hidden]`` scales, all in
    the layout ``matmul_int4`` takes, UNSHARDED (on any device): the constructor keeps only this
    rank's shard, on ``device``.

    ``run(x, m)`` returns the f32 ``[m, hidden]`` output: complete when ``reduce="all"`` (or one
    rank), this rank's ``m/P`` rows (``[m/P, hidden]``) when ``reduce="scatter"``, the un-reduced
    partial when ``reduce="none"``.
    """

    def __init__(self, ops, device, hidden: int, inter: int, w_gate, s_gate, w_up, s_up, w_down, s_down,
                 world: int = 1, rank: int = 0, group=None, max_m: int = 4096, reduce: str = "all"):
        if reduce not in ("all", "scatter", "none", "fused", "overlap"):
            raise ValueError(f"reduce must be 'all', 'scatter', 'none', 'fused' or 'overlap', got {reduce!r}")
        self.ops, self.device, self.group = ops, device, group
        self.hidden, self.inter, self.world, self.rank, self.reduce = hidden, inter, world, rank, reduce
        lo, hi = shard_bounds(inter, world, rank, multiple=GROUP)
        self.i_loc = hi - lo
        dev = torch.device("cuda", device.ordinal) if hasattr(device, "ordinal") else torch.device(device)
        wg = shard_packed_int4(w_gate, hidden, inter, world, rank)
        wu = shard_packed_int4(w_up, hidden, inter, world, rank)
        sg = shard_group_scales(s_gate, hidden, inter, world, rank)
        su = shard_group_scales(s_up, hidden, inter, world, rank)
        w_gu, s_gu = concat_gate_up(wg, sg, wu, su, hidden, self.i_loc)
        self.w_gu, self.s_gu = w_gu.to(dev), s_gu.to(dev)
        self.w_down = k_shard_packed_int4(w_down, inter, hidden, world, rank).to(dev)
        self.s_down = k_shard_group_scales(s_down, inter, hidden, world, rank).contiguous().to(dev)
        self.max_m = max_m
        self.gu = torch.empty(max_m * 2 * self.i_loc, dtype=torch.float16, device=dev)
        self.act = torch.empty(max_m * self.i_loc, dtype=torch.float16, device=dev)
        self.out = torch.empty(max_m * hidden, dtype=torch.float32, device=dev)
        self.rows = torch.empty((max_m // world) * hidden, dtype=torch.float32, device=dev) \
            if (world > 1 and reduce == "scatter") else None
        self.fuse_silu = False
        if world > 1 and reduce == "fused":
            self._init_fused(dev)

    def enable_fused_silu(self, on: bool = True):
        """Run gate|up and the SiLU-gate as ONE launch (``matmul_int4_silu_gate``: the activation in
        the GEMM's epilogue for m > 512, so the ``[m, 2I]`` projection never reaches memory) in
        :meth:`local`, :meth:`run_fused` and :meth:`run_switch`.  Keeps a second, column-interleaved
        copy of the gate|up shard.  The bits do not change."""
        if on and not hasattr(self, "w_gu_il"):
            self.w_gu_il, self.s_gu_il = interleave_gate_up(self.w_gu, self.s_gu, self.hidden, self.i_loc)
        self.fuse_silu = bool(on)

    def _gate_up_act(self, x: torch.Tensor, m: int, mark):
        """``act[m, I_loc] = silu(x W_gate) * (x W_up)`` in ``self.act``: one launch or two."""
        ops, d, il, h = self.ops, self.device, self.i_loc, self.hidden
        if self.fuse_silu:
            ops.matmul_int4_silu_gate(d, x, self.w_gu_il, self.s_gu_il, self.act, self.gu, m, il, h, GROUP)
            mark("gate_up_silu")
            return
        ops.matmul_int4(d, x, self.w_gu, self.s_gu, self.gu, m, 2 * il, h, GROUP)
        mark("gate_up")
        # row r of gu = [gate(r, 0..il) | up(r, 0..il)]
        ops.silu_gate_f16(d, self.gu, self.gu.view(-1)[il:], self.act, m, il, x_ld=2 * il, gate_ld=2 * il)
        mark("silu_gate")

    # ---- reduction fused into the down projection (peer stores + barrier + slot sum)

    #: one step while the bytes it sends beyond a two-step all-reduce cost less than a barrier
    ONE_STEP_EXTRA_BYTES = 6 << 20

    def one_step(self, m: int) -> bool:
        p = self.world
        return (p - 1) * (1.0 - 2.0 / p) * m * self.hidden * 4 <= self.ONE_STEP_EXTRA_BYTES

    def _init_fused(self, dev):
        import torch.distributed._symmetric_memory as symm_mem
        if self.hidden % (self.world * 64) != 0:
            raise ValueError(f"hidden={self.hidden} must split into {self.world} blocks of a multiple of 64 columns")
        group = self.group if self.group is not None else dist.group.WORLD
        self.m_one = max([m for m in range(1, self.max_m + 1) if self.one_step(m)] or [0])
        # [two one-step staging buffers, used alternately][the two-step staging buffer]
        self.one_elems = self.world * self.m_one * self.hidden
        two_elems = self.max_m * self.hidden
        self.stage = symm_mem.empty(2 * self.one_elems + two_elems, dtype=torch.float32, device=dev)
        self.stage_h = symm_mem.rendezvous(self.stage, group)
        self.out_sym = symm_mem.empty(self.max_m * self.hidden, dtype=torch.float32, device=dev)
        self.out_h = symm_mem.rendezvous(self.out_sym, group)
        self.stage_ptrs = [int(p) for p in self.stage_h.buffer_ptrs]
        self.out_ptrs = [int(p) for p in self.out_h.buffer_ptrs]
        self.flip = 0
        # Store-back of the two-step form through the NVLink multicast object torch binds the
        # symmetric output buffers to, where the fabric offers one (0 otherwise): the summed block
        # leaves this GPU once instead of once per peer.  KAIO_B200_MULTICAST=0 keeps peer stores.
        self.out_mc = 0
        if os.environ.get("KAIO_B200_MULTICAST", "1") != "0":
            self.out_mc = int(getattr(self.out_h, "multicast_ptr", 0) or 0)

    def _store_back(self, dev, off: int, rows: int, r0: int = 0):
        """Second step of the two-step form for ``rows`` rows starting at ``r0``: add this rank's
        column block over the P staging slots at ``stage[off:]`` and deliver it to every rank."""
        h, p = self.hidden, self.world
        blk = h // p
        slots = self.stage[off:off + rows * h]
        if self.out_mc:
            self.ops.sum_partials_f32_multicast(dev, slots, p, rows, blk, self.out_mc + r0 * h * 4, rows * h, h,
                                                self.rank * blk)
        else:
            self.ops.sum_partials_f32(dev, slots, p, rows, blk, [q + r0 * h * 4 for q in self.out_ptrs], rows * h, h,
                                      self.rank * blk)

    def run_fused(self, x: torch.Tensor, m: int, mark=None) -> torch.Tensor:
        """gate|up, SiLU-gate, then the down projection whose epilogue stores into the ranks' staging
        slots, the barrier, and the slot sum.  Returns the complete f32 ``[m, hidden]``.
        ``mark(label)``, if given, is called after every launch (stage timing with events)."""
        if m > self.max_m:
            raise ValueError(f"m={m} exceeds max_m={self.max_m}")
        mark = mark or (lambda label: None)
        ops, d, il, h, p = self.ops, self.device, self.i_loc, self.hidden, self.world
        self._gate_up_act(x, m, mark)
        if m <= self.m_one:
            off = self.flip * self.one_elems
            self.flip ^= 1
            ops.matmul_int4_peer_partials(d, self.act, self.w_down, self.s_down, [q + off * 4 for q in self.stage_ptrs],
                                          p * m * h, p, self.rank, False, m, h, il, GROUP)
            mark("down_peer_stores")
            self.stage_h.barrier()  # every rank's partial has landed in every rank's slots
            mark("barrier")
            ops.sum_partials_f32(d, self.stage[off:off + p * m * h], p, m, h, [self.out.data_ptr()], m * h, h, 0)
            mark("slot_sum")
            return self.out[: m * h].view(m, h)
        off = 2 * self.one_elems
        ops.matmul_int4_peer_partials(d, self.act, self.w_down, self.s_down, [q + off * 4 for q in self.stage_ptrs],
                                      m * h, p, self.rank, True, m, h, il, GROUP)
        mark("down_peer_stores")
        self.stage_h.barrier()  # column block r of every rank's partial has landed on rank r
        mark("barrier")
        self._store_back(d, off, m)
        mark("slot_sum_store_back")
        self.out_h.barrier()  # every rank's summed block has landed in every rank's output
        mark("closing_barrier")
        return self.out_sym[: m * h].view(m, h)

    def run_fused_pipelined(self, x: torch.Tensor, m: int, chunks: "list[int] | None" = None) -> torch.Tensor:
        """The two-step fused all-reduce hidden behind the chain itself.  The rows are cut into
        chunks; every chunk runs gate|up (f16 GEMM on weights dequantised once per call), SiLU-gate
        and the down projection whose epilogue scatters the f32 partial tiles to the ranks that own
        the column blocks (peer stores, as in :meth:`run_fused`); while chunk ``i+1`` computes on
        the calling stream, chunk ``i``'s barrier, slot sum (fixed rank order: the same bits on
        every rank and run), store-back to every rank and closing barrier run on a second stream.
        The NVLink traffic of a chunk (2 x (P-1)/P of its f32 partial rows per rank) thus has a
        whole chunk of compute to hide behind; only the last chunk's store-back is exposed.
        Returns the complete f32 ``[m, hidden]`` (symmetric memory) on every rank."""
        if m > self.max_m:
            raise ValueError(f"m={m} exceeds max_m={self.max_m}")
        ops, d, il, h, p = self.ops, self.device, self.i_loc, self.hidden, self.world
        if chunks is None:
            chunks = [m - m // 2, m // 2] if m >= 512 else [m]
        if sum(chunks) != m or min(chunks) < 1:
            raise ValueError(f"chunks {chunks} do not add up to m={m}")
        if not hasattr(self, "side_stream"):
            self.side_stream = torch.cuda.Stream(device=self.out.device)
        if not hasattr(self, "w_gu_f16"):
            self._init_overlap()
        ops.dequantize_int4(d, self.w_gu, self.s_gu, self.w_gu_f16, h, 2 * il, GROUP)
        main = torch.cuda.current_stream()
        base, blk = 2 * self.one_elems, h // p
        side_dev = type(d)(d.ordinal, self.side_stream)
        r0 = 0
        for rows in chunks:
            xs = x.view(-1)[r0 * h:(r0 + rows) * h]
            gu = self.gu[r0 * 2 * il:(r0 + rows) * 2 * il]
            act = self.act[r0 * il:(r0 + rows) * il]
            ops.matmul_tc_f16out(d, xs, self.w_gu_f16, gu, rows, 2 * il, h)
            ops.silu_gate_f16(d, gu, gu[il:], act, rows, il, x_ld=2 * il, gate_ld=2 * il)
            off = base + r0 * h  # this chunk's [P][rows][h/P] staging region (rows * h floats)
            ops.matmul_int4_peer_partials(d, act, self.w_down, self.s_down, [q + off * 4 for q in self.stage_ptrs],
                                          rows * h, p, self.rank, True, rows, h, il, GROUP)
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.side_stream):
                self.side_stream.wait_event(ev)
                self.stage_h.barrier()  # column block r of every rank's partial rows has landed on rank r
                self._store_back(side_dev, off, rows, r0)
                self.out_h.barrier()  # every rank's summed block of these rows has landed everywhere
            r0 += rows
        main.wait_stream(self.side_stream)
        return self.out_sym[: m * h].view(m, h)

    # ---- all-reduce inside the NVSwitch (multimem.ld_reduce + multimem.st)

    def _init_switch(self):
        """Symmetric partial buffer for :meth:`run_switch`; needs the multicast addresses that torch
        symmetric memory hands out where the fabric offers NVLink multicast."""
        import torch.distributed._symmetric_memory as symm_mem
        if not hasattr(self, "out_h"):
            self._init_fused(self.out.device)
        group = self.group if self.group is not None else dist.group.WORLD
        self.part_sym = symm_mem.empty(self.max_m * self.hidden, dtype=torch.float32, device=self.out.device)
        self.part_h = symm_mem.rendezvous(self.part_sym, group)
        self.part_mc = int(getattr(self.part_h, "multicast_ptr", 0) or 0)
        self.out_mc_switch = int(getattr(self.out_h, "multicast_ptr", 0) or 0)
        if not self.part_mc or not self.out_mc_switch:
            raise RuntimeError("no NVLink multicast address for the symmetric buffers on this fabric")
        if not hasattr(self, "side_stream"):
            self.side_stream = torch.cuda.Stream(device=self.out.device)

    def run_switch(self, x: torch.Tensor, m: int, chunks: "list[int] | None" = None, mark=None) -> torch.Tensor:
        """The chain with the all-reduce done by the NVSwitch: every rank writes its f32 partial
        ``[m, hidden]`` into its own symmetric buffer, the ranks meet at a barrier, and rank ``r``
        runs ``allreduce_multimem_f32`` on column block ``r`` -- ``multimem.ld_reduce`` adds the
        eight partial elements inside the switch, ``multimem.st`` delivers the sum to every rank's
        output -- so per rank and direction ``m * hidden * 4`` bytes cross NVLink instead of the
        ``2 (P-1)/P`` times that of the peer-store form.  One reducer per element: the same bits on
        every rank.  With ``chunks`` (row counts) the down projection runs chunk by chunk on
        weights dequantised once, and chunk ``i``'s barrier + in-switch reduction run on a second
        stream under chunk ``i+1``'s GEMM.  Returns the complete f32 ``[m, hidden]`` (symmetric
        memory) on every rank."""
        if m > self.max_m:
            raise ValueError(f"m={m} exceeds max_m={self.max_m}")
        if not hasattr(self, "part_mc"):
            self._init_switch()
        mark = mark or (lambda label: None)
        ops, d, il, h, p = self.ops, self.device, self.i_loc, self.hidden, self.world
        blk = h // p
        chunks = chunks or [m]
        if sum(chunks) != m or min(chunks) < 1:
            raise ValueError(f"chunks {chunks} do not add up to m={m}")
        self._gate_up_act(x, m, mark)
        if len(chunks) == 1:
            ops.matmul_int4(d, self.act, self.w_down, self.s_down, self.part_sym, m, h, il, GROUP)
            mark("down")
            self.part_h.barrier()  # every rank's partial is complete
            mark("barrier")
            ops.allreduce_multimem_f32(d, self.part_mc, self.out_mc_switch, m * h, m, blk, h, self.rank * blk)
            mark("in_switch_all_reduce")
            self.out_h.barrier()  # every block of the output has landed everywhere
            mark("closing_barrier")
            return self.out_sym[: m * h].view(m, h)
        if not hasattr(self, "w_down_f16"):
            self._init_overlap()
        ops.dequantize_int4(d, self.w_down, self.s_down, self.w_down_f16, il, h, GROUP)
        main = torch.cuda.current_stream()
        side_dev = type(d)(d.ordinal, self.side_stream)
        r0 = 0
        for rows in chunks:
            ops.matmul_tc(d, self.act[r0 * il:(r0 + rows) * il], self.w_down_f16,
                          self.part_sym[r0 * h:(r0 + rows) * h], rows, h, il)
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.side_stream):
                self.side_stream.wait_event(ev)
                self.part_h.barrier()
                ops.allreduce_multimem_f32(side_dev, self.part_mc + r0 * h * 4, self.out_mc_switch + r0 * h * 4,
                                           rows * h, rows, blk, h, self.rank * blk)
                self.out_h.barrier()
            r0 += rows
        main.wait_stream(self.side_stream)
        return self.out_sym[: m * h].view(m, h)

    # ---- all-reduce overlapped with the GEMMs (large M)

    @staticmethod
    def default_chunks(m: int) -> list[int]:
        """Row chunks for :meth:`run_overlapped`: about a half, then a third, then the rest, each
        a multiple of 256 rows (the tile height of the paired GEMM) -- the exchange of a chunk
        hides behind the next chunk's GEMMs, and only the last, smallest chunk's is exposed."""
        if m <= 1024 or m % 256 != 0:
            return [m]
        t = m // 256
        first = max(1, t // 2)
        second = max(1, (t - first) * 5 // 8)
        rest = t - first - second
        rows = [first * 256, second * 256] + ([rest * 256] if rest > 0 else [])
        return sorted(rows, reverse=True)

    def _init_overlap(self):
        dev = self.out.device
        self.w_gu_f16 = torch.empty(self.hidden * 2 * self.i_loc, dtype=torch.float16, device=dev)
        self.w_down_f16 = torch.empty(self.i_loc * self.hidden, dtype=torch.float16, device=dev)
        self.comm_stream = torch.cuda.Stream(device=dev)

    def run_overlapped(self, x: torch.Tensor, m: int, chunks: "list[int] | None" = None) -> torch.Tensor:
        """The chain for large ``m`` with its all-reduce hidden behind the GEMMs.

        The weights are dequantised ONCE per call (``dequantize_int4``, the pre-pass that
        ``matmul_int4`` runs internally for m > 512), the rows are cut into ``chunks``, and while
        chunk ``i+1`` runs its three launches (f16 GEMM, SiLU-gate, f16 GEMM) on the calling
        stream, chunk ``i``'s f32 partial rows are summed across the ranks by NCCL on a second
        stream.  Per element this is the arithmetic of :meth:`local` (same kernels, same
        operands), so the un-reduced partial is bit-identical to it.  Returns the complete f32
        ``[m, hidden]`` on every rank."""
        if m > self.max_m:
            raise ValueError(f"m={m} exceeds max_m={self.max_m}")
        if not hasattr(self, "w_gu_f16"):
            self._init_overlap()
        chunks = list(chunks) if chunks is not None else self.default_chunks(m)
        if sum(chunks) != m or min(chunks) < 1:
            raise ValueError(f"chunks {chunks} do not add up to m={m}")
        ops, d, il, h = self.ops, self.device, self.i_loc, self.hidden
        ops.dequantize_int4(d, self.w_gu, self.s_gu, self.w_gu_f16, h, 2 * il, GROUP)
        ops.dequantize_int4(d, self.w_down, self.s_down, self.w_down_f16, il, h, GROUP)
        main = torch.cuda.current_stream()
        r0 = 0
        for rows in chunks:
            xs = x.view(-1)[r0 * h:(r0 + rows) * h]
            gu = self.gu[r0 * 2 * il:(r0 + rows) * 2 * il]
            act = self.act[r0 * il:(r0 + rows) * il]
            out = self.out[r0 * h:(r0 + rows) * h]
            ops.matmul_tc_f16out(d, xs, self.w_gu_f16, gu, rows, 2 * il, h)
            ops.silu_gate_f16(d, gu, gu[il:], act, rows, il, x_ld=2 * il, gate_ld=2 * il)
            ops.matmul_tc(d, act, self.w_down_f16, out, rows, h, il)
            if self.world > 1:
                ev = torch.cuda.Event()
                ev.record(main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(ev)
                    dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
            r0 += rows
        if self.world > 1:
            main.wait_stream(self.comm_stream)
        return self.out[: m * h].view(m, h)

    def local(self, x: torch.Tensor, m: int) -> torch.Tensor:
        """The three launches of this rank; returns the f32 ``[m, hidden]`` partial sum."""
        if m > self.max_m:
            raise ValueError(f"m={m} exceeds max_m={self.max_m}")
        ops, d, il = self.ops, self.device, self.i_loc
        self._gate_up_act(x, m, lambda label: None)
        ops.matmul_int4(d, self.act, self.w_down, self.s_down, self.out, m, self.hidden, il, GROUP)
        return self.out[: m * self.hidden].view(m, self.hidden)

    def run(self, x: torch.Tensor, m: int) -> torch.Tensor:
        if self.world > 1 and self.reduce == "fused":
            return self.run_fused(x, m)
        if self.reduce == "overlap" and m > 512:
            return self.run_overlapped(x, m)
        part = self.local(x, m)
        if self.world == 1 or self.reduce == "none":
            return part
        if self.reduce in ("all", "overlap"):
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
            return part
        if m % self.world != 0:
            raise ValueError(f"reduce='scatter' needs m divisible by the {self.world} ranks, got {m}")
        rows = self.rows[: (m // self.world) * self.hidden].view(m // self.world, self.hidden)
        dist.reduce_scatter_tensor(rows, part, op=dist.ReduceOp.SUM, group=self.group)
        return rows
