"""The bfloat16 kernel set used for serving: a fast kernel where one exists for the shape at
hand, the plain kernel (same arithmetic, bfloat16 storage) otherwise.

Steps of up to 128 rows (decode, short prompts) run the tcgen05 projections that stream the weights once
(``gemv_tc``), with SwiGLU folded into the gate/up projection, and the tensor-core split-key
attention with rotation and cache append inside; prompts run the persistent tcgen05 GEMM and
the tcgen05 flash attention.  Which kernel a shape gets is decided here and nowhere else; the
thresholds are module constants with the measurement that set them beside them."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from . import ops
from .kernel_sets import NormedInput, PlainKernels, as_tensor

TARGET_BLOCKS = 1184           # eight small blocks per SM
DETERMINISTIC_CHUNK_PAGES = 16 # ... and its fixed chunk size (1,024 keys) when results must not depend on the batch
STREAM_ROWS = ops.GEMV_TC_MAX_ROWS   # steps of up to this many rows take the projections that stream the weights once
CLUSTER_CHUNK_PAGES = 8       # the most pages a chunk holds when a sequence's chunks run as a cluster
TC_ATTENTION_MIN_NEW = 96     # prompts at least this long take the tcgen05 attention (tiles of 128 rows)


class FastKernels(PlainKernels):
    name = "fast"
    capturable = True       # no kernel of the set synchronises or allocates: decode steps replay CUDA graphs

    def __init__(self, pdl: bool = True, deterministic: bool = False):
        self.pdl = pdl           # decode kernels launch as programmatic dependents of their predecessors
        # True: no float atomics and one choice of kernel whatever the batch, so that a sequence's
        # logits are the same bits in every run and in every batch (and a sampled sequence is
        # reproducible from its seed): projections never split K, prompts always take the tcgen05
        # attention, the decode attention cuts a sequence's keys in fixed chunks
        self.deterministic = deterministic
        self.fuse_rope = True    # decode attention rotates q/k and appends to the cache itself
        # the prompt's q/k/v projection does so in its epilogue, if the step is large enough for that
        # kernel: not in deterministic mode, where a prompt takes one path whatever accompanies it
        self.fuse_rope_prefill = not deterministic
        self._scratch: Dict[str, torch.Tensor] = {}
        self._zeroed = set()    # names of the buffers that are zero between uses (sums of K parts, arrival counters)
        self._retired = []      # outgrown buffers stay alive: captured graphs still point at them
        ops.after_device_error(self._after_device_error)

    def _after_device_error(self) -> None:
        """A launch gave up on a wait: its arrival counters and partial sums may be left half-way.  The
        buffers that must be zero between uses are zeroed again, so that the steps after the error
        that is about to be raised start from a clean state."""
        for name in self._zeroed:
            t = self._scratch.get(name)
            if t is not None:
                t.zero_()

    def rmsnorm(self, x, weight, eps, out, rows=None):
        pdl = self.pdl and out.shape[0] <= 64
        if ops.rmsnorm_vec_ok(x, weight, out):
            ops.rmsnorm_vec(x, weight, eps, out, rows, pdl=pdl)
        else:
            ops.rmsnorm(x, weight, eps, out, rows, pdl=pdl)

    def rope_append(self, qkv, cos, sin, batch, page_table, k_cache, v_cache, n_q, n_kv, head_dim,
                    rotary_dim, page_shift, write_cache=True):
        if ops.rope_append_vec_ok(qkv, cos, head_dim, rotary_dim, write_cache):
            ops.rope_append_vec(qkv, cos, sin, batch.pos, batch.slot_of_token, page_table, k_cache, v_cache,
                                n_q, n_kv, head_dim, page_shift)
        else:
            super().rope_append(qkv, cos, sin, batch, page_table, k_cache, v_cache, n_q, n_kv, head_dim,
                                rotary_dim, page_shift, write_cache)

    # ---- matrix products -------------------------------------------------------------
    def _skinny(self, x, weight, out, mode) -> bool:
        """The mma.sync skinny GEMM, for up to 64 rows of shapes the tcgen05 kernels refuse."""
        x = as_tensor(x)
        if not ops.skinny_gemm_ok(x, weight):
            return False
        ops.skinny_gemm(x, weight, out, mode, pdl=self.pdl)
        return True

    def linear(self, x, weight, out, accumulate=False):
        rows = x.n_rows if isinstance(x, NormedInput) else x.shape[0]
        x = as_tensor(x)
        if (out.dtype == torch.float32 or not accumulate) and ops.gemm_tc_ok(x, weight, out):
            n, k = weight.shape
            if self.deterministic:
                # one kernel for every row count, K never split: a row's sums are taken in the same order
                # whatever else is in the step (decode steps pay for it: few blocks stream the weights)
                ops.gemm_tc(x, weight, out, ops.TC_ACCUMULATE if accumulate else ops.TC_STORE,
                            tile_n=ops.TC_TILE_PAIR if self._pair_tiles(rows, n) else self._tile_n(rows, n))
            elif rows <= STREAM_ROWS and accumulate:
                # weights on the M side, K split over blocks that add with float atomics
                ops.gemv_tc(x, weight, out, ops.TC_ACCUMULATE, splits=ops.gemv_tc_splits(n, k), pdl=self.pdl)
            elif rows <= STREAM_ROWS and n >= 16384:
                ops.gemv_tc(x, weight, out, ops.TC_STORE, pdl=self.pdl)
            elif rows <= STREAM_ROWS and out.dtype == torch.bfloat16 and n % 8 == 0 and out.stride(0) % 8 == 0:
                # too few row tiles for the SMs (48 for the 8B query/key/value projection): K is split
                # over blocks that add with float atomics into a float32 scratch that is zero between
                # uses; a small kernel rounds the sums into ``out`` and clears the scratch again
                # (batch 64: 22 us of a layer became 11; the ordered sum of parts through scratch
                # that gemv_tc also offers is slower from 9 rows on)
                sums = self._buffer("split_sums", rows * n, torch.float32, out.device, zero=True)[: rows * n].view(rows, n)
                ops.gemv_tc(x, weight, sums, ops.TC_ACCUMULATE, splits=ops.gemv_tc_splits(n, k), pdl=self.pdl)
                ops.round_and_clear(sums, out, pdl=self.pdl)
            else:
                # a prompt of a few hundred tokens: fewer output tiles than SMs.  K is cut into parts
                # that add with float atomics, into the residual or, for a stored result, into the
                # zeroed scratch that round_and_clear turns into bfloat16 (as for decode above)
                tile_n = self._tile_n(rows, n)
                splits = self._gemm_splits(rows, n, k, tile_n)
                if splits == 1 and self._pair_tiles(rows, n):
                    tile_n = ops.TC_TILE_PAIR
                if splits > 1 and accumulate:
                    ops.gemm_tc(x, weight, out, ops.TC_ACCUMULATE, tile_n=tile_n, splits=splits)
                elif splits > 1 and out.dtype == torch.bfloat16 and n % 8 == 0 and out.stride(0) % 8 == 0:
                    sums = self._buffer("split_sums", rows * n, torch.float32, out.device, zero=True)[: rows * n].view(rows, n)
                    ops.gemm_tc(x, weight, sums, ops.TC_ACCUMULATE, tile_n=tile_n, splits=splits)
                    ops.round_and_clear(sums, out, pdl=self.pdl)
                else:
                    ops.gemm_tc(x, weight, out, ops.TC_ACCUMULATE if accumulate else ops.TC_STORE, tile_n=tile_n)
            return
        if rows <= 64 and weight.dtype == torch.bfloat16 and (out.dtype == torch.float32 or not accumulate):
            if self._skinny(x, weight, out, ops.SG_ACCUMULATE if accumulate else ops.SG_STORE):
                return
        ops.gemm_nt_plain(x, weight, out, accumulate)

    @staticmethod
    def _gemm_splits(rows: int, n: int, k: int, tile_n: int, sms: Optional[int] = None) -> int:
        """Parts a tile's K range is cut into so that the work items fill the SMs once (one block
        per SM walks them); at least 8 k-blocks (512 columns) a part; 1 when the tiles alone do."""
        tiles = ((rows + 127) // 128) * ((n + tile_n - 1) // tile_n)
        return max(1, min((sms or ops.sm_count()) // tiles, (k // 64) // 8, 16))

    @staticmethod
    def _pair_tiles(rows: int, n: int) -> bool:
        """Tiles of 256 x 256 on SM pairs: each SM fetches a third less per k-block than with a
        128 x 256 tile of its own, and L2-to-shared-memory bandwidth is what bounds these products
        (2,048 rows of the 8B shapes: 374 to 347 us gate/up, 202 to 184 down, 89 to 79 q/k/v, 72 to
        62 o).  Not where the second half of the last 256 rows would be mostly padding."""
        return n >= 256 and (rows >= 1024 or ((rows + 127) // 128) % 2 == 0)

    @staticmethod
    def _tile_n(rows: int, n: int) -> int:
        """Output-tile width of the tcgen05 GEMM: wide tiles for prefill, narrow ones for a
        handful of rows so that enough blocks stream the weights (measured on 8B shapes)."""
        if rows > 64:
            return 256 if n > 128 else 128
        return 256 if n >= 16384 else 64

    def pack_gate_up(self, gate, up):
        inter = gate.shape[0]
        if inter % 8 or gate.dtype != torch.bfloat16:
            return super().pack_gate_up(gate, up)
        both = torch.stack([gate.view(inter // 8, 8, -1), up.view(inter // 8, 8, -1)], dim=1)
        return both.reshape(2 * inter, -1).contiguous(), "interleaved"      # [8 gate | 8 up] per 16 rows

    def gate_up_swiglu(self, x, w_gate_up, layout, out):
        rows = x.n_rows if isinstance(x, NormedInput) else x.shape[0]
        if layout == "interleaved":
            xt = as_tensor(x)
            if w_gate_up.shape[0] % 16 == 0 and ops.gemm_tc_ok(xt, w_gate_up, out):
                if rows <= STREAM_ROWS and not self.deterministic:
                    ops.gemv_tc(xt, w_gate_up, out, ops.TC_SWIGLU, pdl=self.pdl)
                else:
                    n2 = w_gate_up.shape[0]
                    ops.gemm_tc(xt, w_gate_up, out, ops.TC_SWIGLU,
                                tile_n=ops.TC_TILE_PAIR if self._pair_tiles(rows, n2) else self._tile_n(rows, n2))
                return
        if layout == "interleaved" and rows <= 64 and self._skinny(x, w_gate_up, out, ops.SG_SWIGLU):
            return
        super().gate_up_swiglu(x, w_gate_up, layout, out)

    # ---- attention -------------------------------------------------------------------
    def _buffer(self, name: str, n: int, dtype, device, zero=False) -> torch.Tensor:
        t = self._scratch.get(name)
        if t is None or t.numel() < n or t.device != device:
            if t is not None:
                self._retired.append(t)
            t = (torch.zeros if zero else torch.empty)(max(n, 4096), dtype=dtype, device=device)
            self._scratch[name] = t
        if zero:
            self._zeroed.add(name)
        return t

    def _chunks(self, n_kv: int, pages: int, blocks: int):
        """(pages per chunk, most chunks of one sequence) for the tensor-core decode attention over a batch
        whose longest sequence spans up to ``pages``.  Normally the kernel sizes the chunks itself from
        the batch's real lengths (0): a work item has a fixed cost of about six pages' worth of
        streaming, so items should be as large as still fills the ``blocks`` the device holds; what is
        decided here is only how much scratch that can need: a sequence is never cut finer than two
        pages a chunk, nor into more chunks than there are blocks for its kv heads.  In deterministic
        mode the chunk is a constant, so that a sequence is cut the same way in every batch."""
        if self.deterministic:
            return DETERMINISTIC_CHUNK_PAGES, -(-pages // DETERMINISTIC_CHUNK_PAGES)
        return 0, max(1, min(-(-pages // 2), blocks // max(n_kv, 1) + 1))

    def _cluster(self, heads: int, pages: int, blocks: int) -> int:
        """Chunks a sequence (0: none) when the chunks of a (sequence, kv head) run as a thread-block
        cluster that merges through its shared memory instead of scratch and a counter in L2.  For
        batches so small that ``heads`` (sequences x kv heads) times the chunks is at most one block an
        SM (more blocks keep the next projection's blocks from becoming resident early: batch 4 with 256
        blocks lost 4 % of a step, with 128 it is even), and chunks of at most CLUSTER_CHUNK_PAGES pages
        (one block streams a chunk's pages one after another).  Measured at 8B sizes with 512 keys, a
        step of 16 layers: batch 1 1,566 to 1,509 us, batch 2 1,564 to 1,531, batch 8 1,634 to 1,621."""
        if self.deterministic:
            return 0
        for c in (8, 4, 2):
            if heads * c <= min(blocks, ops.sm_count()):
                return c if pages <= CLUSTER_CHUNK_PAGES * c else 0
        return 0

    def _decode_attention(self, q, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim,
                          page_shift, window, scale, cos=None, sin=None):
        group = n_q // n_kv
        # the bucket's upper end: the most pages a sequence of this batch can span
        pages = 2 * batch.kv_pages - 1 if batch.kv_pages > 1 else 1
        if window:
            pages = min(pages, (window >> page_shift) + 2)
        if ops.attention_decode_chunked_ok(batch.n_seqs, n_q, n_kv, head_dim, q.stride(0), page_shift):
            # tensor-core kernel on a persistent grid (beside the mma.sync skinny GEMM it made a step
            # slower: the two compete for the SM's L1/shared memory; beside the tcgen05 projections it
            # is the faster choice at every batch size: batch 16: 4.24 to 3.57 ms a step)
            blocks = ops.attention_decode_chunked_blocks(batch.n_seqs, n_q, n_kv, head_dim, cos is not None)
            chunk, max_chunks = self._chunks(n_kv, pages, blocks)
            cluster = self._cluster(batch.n_seqs * n_kv, pages, blocks)
            if cluster and batch.n_seqs * n_kv > ops.attention_decode_chunked_clusters(n_q, n_kv, head_dim, cos is not None, cluster):
                cluster = 0                              # the device cannot hold that many clusters of this kernel at once
            scratch = counters = None
            if max_chunks > 1 and not cluster:
                nf, nc = ops.attention_decode_chunked_scratch(batch.n_seqs, n_q, n_kv, head_dim, max_chunks)
                scratch = self._buffer("attn_partials", nf, torch.float32, q.device)
                counters = self._buffer("attn_counters", nc, torch.int32, q.device, zero=True)
            ops.attention_decode_chunked(q, k_cache, v_cache, batch.pos, batch.slot_of_token, page_table, out,
                                         n_q, n_kv, head_dim, page_shift, window, scale, chunk, max_chunks,
                                         scratch, counters, pdl=self.pdl, cos=cos, sin=sin, cluster=cluster)
            return
        blocks = batch.n_seqs * n_kv * ((group + 3) // 4)
        if self.deterministic:
            n_splits = 1                                                  # one order of the keys whatever the batch
        elif batch.n_seqs <= 2:
            n_splits = max(1, min(TARGET_BLOCKS // blocks, pages, 16))    # latency-bound: a page a block
        elif pages < 32:
            n_splits = min(2, pages)                                      # measured best for 3..31 sequences
        else:
            n_splits = max(1, min(TARGET_BLOCKS // blocks, pages, 64))
        scratch = counters = None
        if n_splits > 1:
            nf, nc = ops.attention_decode_scratch(batch.n_seqs, n_q, n_kv, head_dim, n_splits)
            scratch = self._buffer("attn_partials", nf, torch.float32, q.device)
            counters = self._buffer("attn_counters", nc, torch.int32, q.device, zero=True)
        ops.attention_decode(q, k_cache, v_cache, batch.pos, batch.slot_of_token, page_table, out,
                             n_q, n_kv, head_dim, page_shift, window, scale, n_splits, scratch, counters,
                             pdl=self.pdl, cos=cos, sin=sin)

    def project_rope_append(self, x, w_qkv, qkv, position, kv, batch, n_q, n_kv, head_dim, page_shift) -> bool:
        """Prompts whose tiles alone fill the SMs: the tcgen05 projection rotates q and k from its
        float32 sums and writes k and v into the cache (no separate rope + append launch, and the
        key and value columns never go through ``qkv``)."""
        tables = getattr(position, "rotary_tables", None)
        rows = batch.n_tokens
        if not (self.fuse_rope_prefill and tables and not batch.is_decode and rows > 64
                and w_qkv.dtype == torch.bfloat16 and head_dim in (64, 128)):
            return False
        n, k = w_qkv.shape
        if self._gemm_splits(rows, n, k, 256) > 1:
            return False                      # a short prompt: K split over blocks is the faster way
        cos, sin, rotary_dim = tables()
        k_cache, v_cache, page_table, _ = kv
        x = as_tensor(x)
        if rotary_dim != head_dim or not ops.gemm_tc_ok(x, w_qkv, qkv) or k_cache.dtype != torch.bfloat16:
            return False
        position.check_range(batch)
        ops.gemm_tc_rope_append(x, w_qkv, qkv, cos, sin, batch.pos, batch.slot_of_token, page_table, k_cache,
                                v_cache, n_q, n_kv, head_dim, page_shift,
                                tile_n=ops.TC_TILE_PAIR if self._pair_tiles(rows, n) else 256)
        return True

    def rope_attention(self, qkv, position, kv, batch, out, n_q, n_kv, head_dim, page_shift, window,
                       scale) -> bool:
        tables = getattr(position, "rotary_tables", None)
        if not (self.fuse_rope and batch.is_decode and tables and qkv.dtype == torch.bfloat16
                and head_dim in (32, 64, 128, 256) and qkv.stride(0) % 8 == 0):
            return False
        cos, sin, rotary_dim = tables()
        if rotary_dim != head_dim:
            return False
        position.check_range(batch)
        k_cache, v_cache, page_table, _ = kv
        self._decode_attention(qkv, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim,
                               page_shift, window, scale, cos, sin)
        return True

    def attention(self, q, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim, page_shift,
                  window: Optional[int], scale: float):
        if batch.is_decode and q.dtype == torch.bfloat16 and head_dim <= 256 and head_dim % 16 == 0 \
                and q.stride(0) % 8 == 0:
            self._decode_attention(q, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim,
                                   page_shift, window, scale)
            return
        if not batch.is_decode and (batch.max_new >= TC_ATTENTION_MIN_NEW or self.deterministic) and k_cache.is_contiguous() \
                and v_cache.is_contiguous() and ops.attention_prefill_tc_ok(q, out, head_dim, page_shift):
            ops.attention_prefill_tc(q, k_cache, v_cache, batch.cu_new, batch.seq_start, batch.seq_slot,
                                     page_table, out, batch.max_new, n_q, n_kv, head_dim, page_shift, window, scale)
            return
        if not batch.is_decode and ops.attention_prefill_ok(q, head_dim) and out.stride(0) % 2 == 0:
            ops.attention_prefill(q, k_cache, v_cache, batch.cu_new, batch.seq_start, batch.seq_slot,
                                  page_table, out, batch.max_new, n_q, n_kv, head_dim, page_shift, window, scale)
            return
        super().attention(q, k_cache, v_cache, batch, page_table, out, n_q, n_kv, head_dim, page_shift,
                          window, scale)
