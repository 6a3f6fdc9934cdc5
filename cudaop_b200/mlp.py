"""Tensor-parallel SwiGLU MLP on FP8 weights — one process per GPU.

Same decomposition as the reference's ``nccl_mlp_test`` (op/nccl/nccl_mlp_test.cu:144-196,321-352):
the first projection is split by output features (column-parallel, no communication), the second
by input features (row-parallel), the input is replicated, and one sum all-reduce of the partial
outputs leaves identical replicas on every rank.  Differences that the benchmark configuration
asks for: SwiGLU instead of GELU, E4M3 weights with one fp32 scale per output channel, bf16
activations quantised per token, and 1/2/4/8 ranks (``torch.distributed``, NCCL over NVLink)
instead of two devices driven by one host thread.

Per rank and forward pass:
  1. quantise X (bf16) per token           -> Xq (E4M3), sx            [b200q_quant_rows_e4m3]
  2. gate/up GEMM + SwiGLU, fused epilogue -> H  (bf16) [T, I/R]       [b200q_gemm_fp8_swiglu]
  3. quantise H per token                  -> Hq (E4M3), sh            [b200q_quant_rows_e4m3]
  4. down GEMM, per-token x per-channel    -> partial Y                [b200q_gemm_fp8_rowcol]
  5. R > 1: sum all-reduce of the fp32 partials.  ``comm="fused"`` (default): step 4 and the
     all-reduce are ONE kernel (b200q_gemm_fp8_rowcol_allreduce) — finished row groups are summed
     in the NVSwitch (multimem.ld_reduce), rounded once to bf16 and broadcast (multimem.st) while
     later groups are still being multiplied.  ``comm="symm"``: the stand-alone NVSwitch kernel
     (b200q_allreduce_to_bf16) per token chunk on a side stream; ``comm="nccl"``:
     torch.distributed.all_reduce + a cast.  All three keep fp32 accumulation and identical replicas.
     ``comm="pipelined"``: as "symm" with one chunk, but forward() does not wait for the all-reduce:
     it runs on the side stream under the NEXT forward's GEMMs (independent batches), partials and
     outputs double-buffered; the caller orders its use of Y after ``output_ready`` (an event) or
     calls ``wait()``.  Throughput mode for a stream of batches; "fused" is the latency mode.

Every cross-rank wait inside the kernels is bounded (b200q_set_wait_limit_ms, 10 s by default).  A
kernel that gives up returns early and leaves an UNDEFINED result; nothing in forward() can see
that without synchronising, so callers that need the guarantee call ``check()`` (it synchronises
and raises ``cudaop_b200.WaitTimeout``) before they trust Y — once per step, or per batch of steps.
"""
from __future__ import annotations

import warnings

import torch

import cudaop_b200 as ops


def shard_mlp_weights(w_gate, s_gate, w_up, s_up, w_down, s_down, rank: int, world: int):
    """Returns this rank's shard of every weight (works on CPU or CUDA tensors).

    w_gate / w_up are [I, H] (K-contiguous, output feature = row): rank r keeps rows
    [r*I/R, (r+1)*I/R) and the matching gate/up scales — the output-feature split of
    op/nccl/nccl_mlp_test.cu:321-340 in the [out, in] layout.  w_down is [H, I]: rank r keeps
    input features (columns) [r*I/R, (r+1)*I/R), re-packed contiguously; its per-output-channel
    scales are not split — the input-feature split of op/nccl/nccl_mlp_test.cu:342-352.
    """
    I = w_gate.shape[0]
    if I % world != 0:
        raise ValueError(f"intermediate size {I} is not divisible by {world} ranks")
    loc = I // world
    lo, hi = rank * loc, (rank + 1) * loc
    return (w_gate[lo:hi].contiguous(), s_gate[lo:hi].contiguous(),
            w_up[lo:hi].contiguous(), s_up[lo:hi].contiguous(),
            w_down[:, lo:hi].contiguous(), s_down.contiguous())


def copy_exchange_plan(rank: int, world: int, elems: int):
    """The copy-engine exchange of `elems` output elements as plain index ranges (no device needed).

    Returns ``(mine, pulls_partial, pulls_result)``: rank r owns ``mine = (r*n/R, (r+1)*n/R)``; first it copies
    that range of every peer's partial sums to itself (``pulls_partial``: peers in the order r+1, r+2, ... so that at
    any moment the ranks read from different peers), adds the R contributions in rank order, and then copies
    every peer's own range of the result (``pulls_result``: ``(peer, lo, hi)``).  Mirrors the two phases of the
    ncclAllReduce in op/nccl/nccl_mlp_test.cu:181-195 (reduce-scatter, all-gather)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank/world out of range")
    if elems % (8 * world) != 0:
        raise ValueError("the element count must be divisible by 8 * world")
    per = elems // world
    order = [(rank + d) % world for d in range(1, world)]
    mine = (rank * per, (rank + 1) * per)
    return mine, [(r, mine[0], mine[1]) for r in order], [(r, r * per, (r + 1) * per) for r in order]


class TensorParallelMLP:
    """Y = down( silu(X Wg^T) * (X Wu^T) ), weights E4M3 with per-output-channel scales."""

    def __init__(self, w_gate, s_gate, w_up, s_up, w_down, s_down, rank: int = 0, world: int = 1,
                 group=None, device=None, max_tokens: int = 4096, chunks: int | None = None,
                 presharded: bool = False, comm: str = "auto", ar_ctas: int | None = None, partial_dtype=torch.bfloat16,
                 use_multicast: bool | None = None):
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if presharded:      # the caller already holds only this rank's shard
            sh = (w_gate, s_gate, w_up, s_up, w_down, s_down)
        else:
            sh = shard_mlp_weights(w_gate, s_gate, w_up, s_up, w_down, s_down, rank, world)
        (self.wg, self.sg, self.wu, self.su, self.wd, self.sd) = [t.to(self.device) for t in sh]
        self.hidden = self.wg.shape[1]
        self.inter_local = self.wg.shape[0]
        self.max_tokens = max_tokens
        self.chunks = chunks if chunks is not None else (1 if world == 1 else 4)
        T, H, Il = max_tokens, self.hidden, self.inter_local
        dev = self.device
        # workspaces: allocated once, reused by every forward
        self.xq = torch.empty((T, H), dtype=torch.uint8, device=dev)
        self.sx = torch.empty((T,), dtype=torch.float32, device=dev)
        # prepare(): the next batch's activations are quantised on a side stream while this batch's GEMMs run
        self._prep_stream = None
        self._prep = None             # (data_ptr, tokens, slot) of the batch prepare() has quantised
        self._prep_slot = 0
        self._prep_xq, self._prep_sx = [None, None], [None, None]
        self._prep_ready, self._prep_free = [None, None], [None, None]
        self.h = torch.empty((T, Il), dtype=torch.bfloat16, device=dev)
        self.hq = torch.empty((T, Il), dtype=torch.uint8, device=dev)
        self.shs = torch.empty((T,), dtype=torch.float32, device=dev)
        self.partial = None
        self.comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None
        self.comm = "none"
        self.ar_ctas = ar_ctas
        # Partial outputs travel as bf16 by default (half the NVLink bytes; the all-reduce then is
        # "fp32 sum of the ranks' bf16 partials, one rounding"); torch.float32 keeps the reference's
        # ncclFloat behaviour exactly.  Transport: plain peer loads/stores (sum in rank order, round to
        # nearest even: bit-reproducible) up to 2 ranks; from 4 ranks on the in-switch reduction
        # (multimem) unless told otherwise: measured 0.43 vs 0.51 ms per step at 8 ranks, at the price
        # that the switch, not this code, rounds the bf16 sum (up to 1 ulp from round-to-nearest-even,
        # still identical on every rank).
        if use_multicast is None:
            use_multicast = world >= 4
        if partial_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("partial_dtype must be torch.bfloat16 or torch.float32")
        self.partial_dtype = partial_dtype
        self.use_multicast = use_multicast
        self._epoch = 0
        if world > 1:
            self.comm = comm
            if comm in ("auto", "fused", "symm", "pipelined", "pipelined_ce", "pipelined_copy"):
                try:
                    self._nbuf = 2 if comm.startswith("pipelined") else 1
                    self._copy_mode = comm == "pipelined_copy"
                    self._init_symmetric(T, H)
                    self.comm = comm if comm in ("symm", "pipelined", "pipelined_ce", "pipelined_copy") else "fused"
                except Exception as exc:
                    if comm != "auto":
                        raise
                    warnings.warn(f"symmetric memory is not available ({type(exc).__name__}: {exc}); "
                                  "the all-reduce falls back to NCCL on fp32 partials")
                    self.comm = "nccl"
            if self.comm in ("fused", "pipelined", "pipelined_ce", "pipelined_copy"):
                self.chunks = 1
            self._buf = 0
            self._ar_done = [None, None]
            self.output_ready = None
            if self.comm == "nccl":
                # NCCL rounds after every hop of its ring when it sums bf16, so this mode always moves fp32
                # partials: fp32 accumulation and one rounding, as in the other modes
                self.partial_dtype = torch.float32
                self.partial = torch.empty((T, H), dtype=torch.float32, device=dev)
        self.kernel_launches_per_forward = 0
        self.top_kernel_events = None     # set to a list to collect (start, end) events of the gate/up kernel
        self.stage_events = None          # set to a list to collect 5 events bracketing the 4 kernels of a stage

    def _init_symmetric(self, T, H):
        """Partial sums, output and barrier flags in symmetric memory (peer-mapped on every rank,
        with an NVSwitch multicast mapping when the fabric offers one)."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = self.group if self.group is not None else dist.group.WORLD
        dev = self.device
        nb = getattr(self, "_nbuf", 1)
        self._partial_all = symm.empty((nb, T, H), dtype=self.partial_dtype, device=dev)
        self._y_all = symm.empty((nb, T, H), dtype=torch.bfloat16, device=dev)
        self.partial = self._partial_all[0]
        self.y_sym = self._y_all[0]
        self._fused_flag_offset = ops.lib().b200q_allreduce_signal_bytes()
        self._bar_offset = self._fused_flag_offset + ops.lib().b200q_fused_allreduce_flag_bytes()
        nflags = (self._bar_offset + ops.lib().b200q_rank_barrier_signal_bytes()) // 4
        self._counters = torch.zeros((ops.lib().b200q_fused_allreduce_counter_bytes() // 4,), dtype=torch.int32, device=dev)
        self.flags = symm.empty((nflags,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        self._hp = symm.rendezvous(self._partial_all, group)
        self._hy = symm.rendezvous(self._y_all, group)
        self._hf = symm.rendezvous(self.flags, group)
        self.multicast = self.use_multicast and bool(self._hp.multicast_ptr) and bool(self._hy.multicast_ptr)
        # every peer's output buffers as tensors this rank can copy from (copy-engine half of "pipelined_ce")
        self._y_peer = [self._hy.get_buffer(r, (nb, T, H), torch.bfloat16, 0) if r != self.rank else None
                        for r in range(self.world)]
        self._p_peer = [self._hp.get_buffer(r, (nb, T, H), self.partial_dtype, 0) if r != self.rank else None
                        for r in range(self.world)]
        self._ce_streams = [torch.cuda.Stream(device=dev) for _ in range(min(4, self.world - 1))]
        self._bar_epoch = 0
        self._stage_buf = None        # "pipelined_copy": the peers' partial sums of this rank's part, brought here by copies
        # launch shape of the stand-alone all-reduce kernel, from measurements at 2/4/8 ranks: the
        # in-switch reduction saturates with few threads (and then disturbs a co-running GEMM least),
        # peer loads need many requests in flight from every SM
        L = ops.lib()
        if getattr(self, "_copy_mode", False) and self.ar_ctas is None:
            self.ar_ctas = 32                   # the local sum kernel: 64 MB of local reads at most
        if self.multicast:
            L.b200q_allreduce_set_threads(256); L.b200q_allreduce_set_unroll(4)
            if self.ar_ctas is None:
                self.ar_ctas = 32
        else:
            L.b200q_allreduce_set_threads(128); L.b200q_allreduce_set_unroll(8)
            if self.ar_ctas is None:
                self.ar_ctas = 148
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def _allreduce_chunk(self, lo, hi, buf: int = 0):
        """Launches the all-reduce kernel for tokens [lo, hi) of buffer `buf` on the current stream."""
        self._epoch += 1
        H = self.hidden
        lo += buf * self.max_tokens
        hi += buf * self.max_tokens
        mc_p = self._hp.multicast_ptr if self.multicast else None
        mc_y = self._hy.multicast_ptr if self.multicast else None
        ops._raise(ops.lib().b200q_allreduce_to_bf16(
            self._hp.buffer_ptrs_dev, self._hy.buffer_ptrs_dev, self._hf.buffer_ptrs_dev, mc_p, mc_y,
            int(self.partial_dtype == torch.bfloat16), lo * H, (hi - lo) * H, self.rank, self.world, self._epoch, 0, self.ar_ctas,
            torch.cuda.current_stream().cuda_stream), "b200q_allreduce_to_bf16")

    def _stage(self, x, y, lo, hi):
        """Steps 1-4 for tokens [lo, hi) on the current stream; returns the number of launches."""
        L = ops.lib(); st = torch.cuda.current_stream().cuda_stream
        n = hi - lo
        H, Il = self.hidden, self.inter_local
        xq, sx, h, hq, shs = self.xq[lo:hi], self.sx[lo:hi], self.h[lo:hi], self.hq[lo:hi], self.shs[lo:hi]
        pre = self._take_prepared(x, lo, hi)
        marks = [] if self.stage_events is not None else None

        def mark():
            if marks is not None:
                e = torch.cuda.Event(enable_timing=True); e.record(); marks.append(e)
        mark()
        if pre is None:
            ops._raise(L.b200q_quant_rows_e4m3(x[lo:hi].data_ptr(), xq.data_ptr(), sx.data_ptr(), n, H, st), "quant x")
        else:                         # quantised ahead of time by prepare(): wait for that kernel, read its buffers
            torch.cuda.current_stream().wait_event(self._prep_ready[pre])
            xq, sx = self._prep_xq[pre][:n], self._prep_sx[pre][:n]
        mark()
        ev = self.top_kernel_events
        if ev is not None:
            e0 = torch.cuda.Event(enable_timing=True); e0.record()
        ops._raise(L.b200q_gemm_fp8_swiglu(xq.data_ptr(), self.wg.data_ptr(), self.wu.data_ptr(), h.data_ptr(),
                                           n, Il, H, sx.data_ptr(), self.sg.data_ptr(), self.su.data_ptr(), st),
                   "gate/up")
        if ev is not None:
            e1 = torch.cuda.Event(enable_timing=True); e1.record()
            ev.append((e0, e1))
        if pre is not None:           # the slot may be overwritten once this GEMM has read it
            free = torch.cuda.Event(); free.record()
            self._prep_free[pre] = free
        mark()
        ops._raise(L.b200q_quant_rows_e4m3(h.data_ptr(), hq.data_ptr(), shs.data_ptr(), n, Il, st), "quant h")
        mark()
        if self.world == 1:
            ops._raise(L.b200q_gemm_fp8_rowcol(hq.data_ptr(), self.wd.data_ptr(), y[lo:hi].data_ptr(), n, H, Il,
                                               shs.data_ptr(), self.sd.data_ptr(), 0, st), "down")
        elif self.comm == "fused":
            if lo != 0:
                raise ValueError("the fused all-reduce covers the whole token range in one call")
            self._epoch += 1
            mc_p = self._hp.multicast_ptr if self.multicast else None
            mc_y = self._hy.multicast_ptr if self.multicast else None
            ops._raise(L.b200q_gemm_fp8_rowcol_allreduce(
                hq.data_ptr(), self.wd.data_ptr(), self.partial.data_ptr(), n, H, Il, shs.data_ptr(), self.sd.data_ptr(),
                self._hp.buffer_ptrs_dev, self._hy.buffer_ptrs_dev, self._hf.buffer_ptrs_dev, mc_p, mc_y,
                int(self.partial_dtype == torch.bfloat16), self._counters.data_ptr(), self._fused_flag_offset, self._epoch, self.rank, self.world, st),
                "down + all-reduce")
        else:
            ops._raise(L.b200q_gemm_fp8_rowcol(hq.data_ptr(), self.wd.data_ptr(), self.partial[lo:hi].data_ptr(),
                                               n, H, Il, shs.data_ptr(), self.sd.data_ptr(),
                                               int(self.partial_dtype == torch.float32), st), "down")
        mark()
        if marks is not None:
            self.stage_events.append(marks)
        return 4

    def prepare(self, x: torch.Tensor, ready: "torch.cuda.Event | None" = None):
        """Quantises the NEXT batch's activations now, on a side stream, so that the kernel runs beside the GEMMs
        already enqueued instead of in front of the next forward().  `x` must be complete when `ready` fires (None:
        it already is — the side stream does not wait for the current stream) and must not change until the
        forward(x) that consumes it has been issued; that forward recognises the batch by its address and size.
        Independent batches only: the reference's benchmark loop (op/nccl/nccl_mlp_test.cu:483-526) is of that kind."""
        ops._check(x, "x", (torch.bfloat16,), 2)
        T, H = x.shape
        if H != self.hidden or T > self.max_tokens:
            raise ValueError(f"x must be [<= {self.max_tokens}, {self.hidden}]")
        with torch.cuda.device(self.device):
            if self._prep_stream is None:
                self._prep_stream = torch.cuda.Stream(device=self.device)
                for i in range(2):
                    self._prep_xq[i] = torch.empty((self.max_tokens, H), dtype=torch.uint8, device=self.device)
                    self._prep_sx[i] = torch.empty((self.max_tokens,), dtype=torch.float32, device=self.device)
            slot = self._prep_slot
            self._prep_slot ^= 1
            ps = self._prep_stream
            if ready is not None:
                ps.wait_event(ready)
            if self._prep_free[slot] is not None:
                ps.wait_event(self._prep_free[slot])
            ops._raise(ops.lib().b200q_quant_rows_e4m3(x.data_ptr(), self._prep_xq[slot].data_ptr(), self._prep_sx[slot].data_ptr(),
                                                       T, H, ps.cuda_stream), "quant x (prepare)")
            ev = torch.cuda.Event(); ev.record(ps)
            self._prep_ready[slot] = ev
            self._prep = (x.data_ptr(), T, slot)

    def cancel_prepared(self):
        """Forgets a batch that prepare() quantised and no forward() has consumed."""
        self._prep = None

    def _take_prepared(self, x, lo, hi):
        """The slot prepare() filled for exactly this batch (whole token range), or None."""
        if self._prep is None:
            return None
        ptr, T, slot = self._prep
        if ptr != x.data_ptr() or lo != 0 or hi != T or x.shape[0] != T:
            return None
        self._prep = None
        return slot

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        ops._check(x, "x", (torch.bfloat16,), 2)
        T, H = x.shape
        if H != self.hidden or T > self.max_tokens:
            raise ValueError(f"x must be [<= {self.max_tokens}, {self.hidden}]")
        if self.comm in ("pipelined", "pipelined_ce", "pipelined_copy"):
            return self._forward_pipelined(x, T)
        if self.comm in ("symm", "fused"):
            y = self.y_sym[:T]
        else:
            y = out if out is not None else torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
        launches = 0
        with torch.cuda.device(self.device):
            if self.world == 1 or self.comm == "fused":
                launches += self._stage(x, y, 0, T)
                if out is not None and self.comm == "fused":
                    out[:T].copy_(y)
                    y = out
            else:
                import torch.distributed as dist
                main = torch.cuda.current_stream()
                nch = max(1, min(self.chunks, T))
                bounds = [T * i // nch for i in range(nch + 1)]
                self.comm_stream.wait_stream(main)
                for c in range(nch):
                    lo, hi = bounds[c], bounds[c + 1]
                    if hi == lo:
                        continue
                    launches += self._stage(x, y, lo, hi)
                    done = torch.cuda.Event(); done.record(main)
                    with torch.cuda.stream(self.comm_stream):
                        self.comm_stream.wait_event(done)
                        if self.comm == "symm":
                            self._allreduce_chunk(lo, hi)
                            launches += 1
                        else:
                            dist.all_reduce(self.partial[lo:hi], op=dist.ReduceOp.SUM, group=self.group)
                            y[lo:hi].copy_(self.partial[lo:hi])     # (fp32 ->) bf16, round-to-nearest-even
                main.wait_stream(self.comm_stream)
                if self.comm == "symm" and out is not None:
                    out[:T].copy_(y)
                    y = out
        self.kernel_launches_per_forward = launches
        return y

    def _forward_pipelined(self, x, T):
        """GEMMs on the current stream, all-reduce on the side stream; returns this step's output
        buffer, which is complete once ``self.output_ready`` has fired."""
        b = self._buf
        self._buf ^= 1
        main = torch.cuda.current_stream()
        with torch.cuda.device(self.device):
            if self._ar_done[b] is not None:            # the all-reduce that last read partial[b] / wrote y[b]
                main.wait_event(self._ar_done[b])
            self.partial = self._partial_all[b]
            launches = self._stage(x, None, 0, T)
            done = torch.cuda.Event(); done.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(done)
                if self.comm == "pipelined_ce":
                    launches += self._reduce_scatter_then_copies(T, b)
                elif self.comm == "pipelined_copy":
                    launches += self._exchange_by_copies(T, b)
                else:
                    self._allreduce_chunk(0, T, buf=b)
                ev = torch.cuda.Event(); ev.record(self.comm_stream)
            self._ar_done[b] = ev
            self.output_ready = ev
        self.kernel_launches_per_forward = launches + 1
        return self._y_all[b][:T]

    def _barrier(self, stream):
        self._bar_epoch += 1
        ops._raise(ops.lib().b200q_rank_barrier(self._hf.buffer_ptrs_dev, self.rank, self.world, self._bar_epoch,
                                                self._bar_offset, stream.cuda_stream), "b200q_rank_barrier")

    def _pull(self, after, pairs):
        """Device-to-device copies (dst, src) spread over the copy streams, all behind event `after`; the side
        stream then waits for them."""
        cs = self.comm_stream
        for k, (dst, src) in enumerate(pairs):
            st = self._ce_streams[k % len(self._ce_streams)]
            st.wait_event(after)
            with torch.cuda.stream(st):
                dst.copy_(src, non_blocking=True)
        for st in self._ce_streams:
            cs.wait_stream(st)

    def _exchange_by_copies(self, T, b):
        """The whole exchange on copy engines: behind a barrier every rank copies the peers' partial sums of ITS 1/R of
        the output into local staging, a small local kernel adds them in rank order (fp32, one rounding: bit for bit
        the rank-order sum) into its own output buffer, and behind a second barrier the ranks copy each other's
        parts.  No SM moves NVLink traffic; the only kernel beside the GEMMs reads local memory.  Staging is reused
        every step: the copies of step i+1 are ordered behind the sum of step i on the side stream.  Returns the
        number of kernel launches beyond the one the caller counts for the exchange."""
        L = ops.lib(); H = self.hidden; R = self.world
        n = T * H
        (lo, hi), pulls_partial, pulls_result = copy_exchange_plan(self.rank, R, n)
        per = hi - lo
        cs = self.comm_stream
        if self._stage_buf is None or self._stage_buf.shape[1] < per:
            self._stage_buf = torch.empty((R, self.max_tokens * H // R), dtype=self.partial_dtype, device=self.device)
            self._src_tables = {}
        mine_p = self._partial_all[b].view(-1)
        key = (b, per)
        if key not in self._src_tables:        # rank order: the own partial in place, the others from staging
            ptrs = [mine_p[lo:hi].data_ptr() if r == self.rank else self._stage_buf[r, :per].data_ptr() for r in range(R)]
            self._src_tables[key] = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        self._barrier(cs)                      # every rank's down projection of this step has finished
        ready = torch.cuda.Event(); ready.record(cs)
        self._pull(ready, [(self._stage_buf[r, :per], self._p_peer[r][b].view(-1)[a:z]) for r, a, z in pulls_partial])
        y = self._y_all[b].view(-1)
        ops._raise(L.b200q_sum_to_bf16(self._src_tables[key].data_ptr(), R, int(self.partial_dtype == torch.bfloat16),
                                       y[lo:hi].data_ptr(), per, self.ar_ctas, cs.cuda_stream), "b200q_sum_to_bf16")
        self._barrier(cs)                      # every rank's part of the result is complete
        summed = torch.cuda.Event(); summed.record(cs)
        self._pull(summed, [(y[a:z], self._y_peer[r][b].view(-1)[a:z]) for r, a, z in pulls_result])
        return 2                               # two barriers and the sum; the caller counts one exchange kernel itself

    def _reduce_scatter_then_copies(self, T, b):
        """The exchange in two phases on the side stream: a kernel sums this rank's 1/R of the output into its own
        buffer, a barrier over the ranks follows, and the other ranks' parts arrive by device-to-device copies
        (copy engines, no SM time).  A rank overwrites its part of buffer b two steps later, behind the start
        barrier of that step's kernel, which every peer passes only after its own copies of this step.
        Returns the number of extra kernel launches (the barrier)."""
        L = ops.lib(); H = self.hidden
        n = T * H
        if n % (8 * self.world) != 0:
            raise ValueError("tokens * hidden must be divisible by 8 * world")
        cs = self.comm_stream
        self._epoch += 1
        mc_p = self._hp.multicast_ptr if self.multicast else None
        ops._raise(L.b200q_reduce_scatter_to_bf16(
            self._hp.buffer_ptrs_dev, self._hy.buffer_ptrs_dev, self._hf.buffer_ptrs_dev, mc_p,
            int(self.partial_dtype == torch.bfloat16), b * self.max_tokens * H, n, self.rank, self.world, self._epoch, 0,
            self.ar_ctas, cs.cuda_stream), "b200q_reduce_scatter_to_bf16")
        self._bar_epoch += 1
        ops._raise(L.b200q_rank_barrier(self._hf.buffer_ptrs_dev, self.rank, self.world, self._bar_epoch, self._bar_offset,
                                        cs.cuda_stream), "b200q_rank_barrier")
        reduced = torch.cuda.Event(); reduced.record(cs)
        per = n // self.world
        mine = self._y_all[b].view(-1)
        k = 0
        for d in range(1, self.world):                     # start with the next rank, so the pulls spread over the links
            r = (self.rank + d) % self.world
            st = self._ce_streams[k % len(self._ce_streams)]; k += 1
            st.wait_event(reduced)
            with torch.cuda.stream(st):
                mine[r * per:(r + 1) * per].copy_(self._y_peer[r][b].view(-1)[r * per:(r + 1) * per], non_blocking=True)
        for st in self._ce_streams:
            cs.wait_stream(st)
        return 1

    def wait(self):
        """Makes the current stream wait for every all-reduce issued so far (no host synchronisation)."""
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    def check(self):
        """Synchronises this rank's device and raises cudaop_b200.WaitTimeout if any kernel issued so far
        gave up on a bounded wait (a peer that never arrived): the outputs since the last check are then
        undefined.  Clears the status word."""
        self.wait()
        with torch.cuda.device(self.device):
            ops.check_status("TensorParallelMLP")

    __call__ = forward


class HostFedMLP:
    """Feeds a TensorParallelMLP with batches that live in pinned HOST memory and leaves the results there.

    The end-to-end path of a job whose activations arrive from the host: per step every rank copies its
    1/R of X from pinned memory over its own PCIe link, the ranks complete each other's copy of X over
    NVLink, the MLP runs, and every rank writes its 1/R of the (replicated) result back to pinned memory.
    All copies run on their own streams and are double-buffered, so the input copy of step i+1 and the
    output copy of step i-1 overlap the GEMMs of step i.

    With R > 1 the X buffers are symmetric memory.  After its host-to-device copy each rank passes a
    stream-ordered barrier (b200q_rank_barrier: every rank's slice has landed) and then pulls the other
    ranks' slices with plain device-to-device copies (copy engines, no SM time taken from the GEMMs, no
    TMA on peer memory).  The barrier of step i+1 is enqueued behind the pulls of step i, so a rank
    overwrites a slice only after every peer has read it.
    """

    def __init__(self, mlp: TensorParallelMLP, tokens: int, prepare_ahead: bool = True):
        self.mlp, self.tokens = mlp, tokens
        self.prepare_ahead = prepare_ahead
        self.rank, self.world, dev = mlp.rank, mlp.world, mlp.device
        H = mlp.hidden
        if tokens % self.world != 0 or tokens > mlp.max_tokens:
            raise ValueError("tokens must be divisible by the number of ranks and fit the MLP's buffers")
        self.rows = tokens // self.world
        self.lo, self.hi = self.rank * self.rows, (self.rank + 1) * self.rows
        self.copy_in, self.copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self._x_free = [None, None]     # event: the forward that last read X buffer b has been issued
        self._y_read = [None, None]     # event: the copy-out that last read output buffer b has finished
        self._ybuf = ([torch.empty((tokens, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
                      if self.world == 1 else None)
        self._step = 0
        self._epoch = 0
        if self.world == 1:
            self.xbuf = [torch.empty((tokens, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
            return
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = mlp.group if mlp.group is not None else dist.group.WORLD
        self._xsym = symm.empty((2, tokens, H), dtype=torch.bfloat16, device=dev)
        self._flags = symm.empty((ops.lib().b200q_rank_barrier_signal_bytes() // 4,), dtype=torch.int32, device=dev)
        self._flags.zero_()
        self._hx = symm.rendezvous(self._xsym, group)
        self._hf = symm.rendezvous(self._flags, group)
        self.xbuf = [self._xsym[0], self._xsym[1]]
        # peer r's copy of both X buffers, as tensors this rank can copy from
        self._peer = [self._hx.get_buffer(r, (2, tokens, H), torch.bfloat16, 0) if r != self.rank else None
                      for r in range(self.world)]
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def step(self, x_host: torch.Tensor, y_host: torch.Tensor):
        """Enqueues one forward pass: x_host / y_host are pinned [tokens, hidden] bf16 tensors; this rank
        reads rows [lo, hi) of x_host and writes rows [lo, hi) of y_host.  Returns at once; finish()
        orders the current stream after everything issued."""
        mlp, b = self.mlp, self._step & 1
        self._step += 1
        main = torch.cuda.current_stream()
        lo, hi, rows = self.lo, self.hi, self.rows
        with torch.cuda.stream(self.copy_in):
            if self._x_free[b] is not None:
                self.copy_in.wait_event(self._x_free[b])
            self.xbuf[b][lo:hi].copy_(x_host[lo:hi], non_blocking=True)
            if self.world > 1:
                self._epoch += 1
                ops._raise(ops.lib().b200q_rank_barrier(self._hf.buffer_ptrs_dev, self.rank, self.world, self._epoch, 0,
                                                        self.copy_in.cuda_stream), "b200q_rank_barrier")
                for r in range(self.world):
                    if r != self.rank:
                        self.xbuf[b][r * rows:(r + 1) * rows].copy_(self._peer[r][b, r * rows:(r + 1) * rows], non_blocking=True)
            ready = torch.cuda.Event(); ready.record(self.copy_in)
        main.wait_event(ready)
        if self.prepare_ahead:                         # quantise X beside the previous step's GEMMs
            mlp.prepare(self.xbuf[b][:self.tokens], ready=ready)
        pipelined = self.world > 1 and mlp.comm.startswith("pipelined")
        if self.world == 1:
            # the layer writes into one of two buffers of this object, not before the copy-out that last read it is done
            if self._y_read[b] is not None:
                main.wait_event(self._y_read[b])
            y = mlp.forward(self.xbuf[b][:self.tokens], out=self._ybuf[b])
        else:
            # the pipelined modes alternate between two output buffers and order the copy-out themselves (it runs
            # on the exchange's stream); the others have ONE output buffer: the next forward waits for the copy-out
            if not pipelined and self._y_read[0] is not None:
                main.wait_event(self._y_read[0])
            y = mlp.forward(self.xbuf[b][:self.tokens])
        done = torch.cuda.Event(); done.record(main)
        self._x_free[b] = done
        side = mlp.comm_stream if pipelined else self.copy_out
        with torch.cuda.stream(side):                 # ordered after this step's GEMMs (and its all-reduce)
            side.wait_event(done)
            y_host[lo:hi].copy_(y[lo:hi], non_blocking=True)
            read = torch.cuda.Event(); read.record(side)
        self._y_read[b if self.world == 1 else 0] = read

    def finish(self):
        main = torch.cuda.current_stream()
        main.wait_stream(self.copy_in); main.wait_stream(self.copy_out)
        self.mlp.wait()

    bytes_in_per_step = property(lambda self: self.tokens * self.mlp.hidden * 2)
    bytes_out_per_step = property(lambda self: self.tokens * self.mlp.hidden * 2)
