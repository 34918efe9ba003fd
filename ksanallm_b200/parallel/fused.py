"""Symmetric-memory heap and the fused tensor-parallel kernels built on it.

Every rank allocates the same three buffers with ``torch.distributed._symmetric_memory`` (CUDA VMM allocations
mapped into every peer's address space, plus an NVLS multicast mapping when the fabric offers one):

* ``partial``  [max_tokens, H] bf16 - where this rank's row-parallel GEMM writes its un-reduced output,
* ``hbuf``     [max_tokens, H] bf16 - where the owners of each row deposit the reduced + normalised activations,
* ``sig``      uint32 flag words for the epoch-stamped cross-rank barriers,
* ``ll_recv`` / ``ll_recv2``  8-byte words {2 x bf16, epoch} of the two hops of the latency-optimised small-step kernel.

The kernels (csrc/cuda/comm_fused.cu) issue the NVLink traffic themselves (``multimem.ld_reduce`` / ``multimem.st``
or plain peer loads/stores); NCCL is only the bootstrap and the measured baseline. Reference counterparts:
NVLS setup in src/ksana_llm/utils/nvidia/cuda_utils.cpp:89-254 and the custom all-reduce buffers registered in
src/ksana_llm/layers/nvidia/custom_all_reduce_sum_layer.cpp:19-104.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import cuda as kcuda


class FusedComm:
    def __init__(self, group, rank: int, size: int, device: torch.device, hidden: int, max_tokens: int,
                 use_multicast: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.size, self.device = rank, size, device
        self.hidden, self.max_tokens = hidden, max_tokens
        self.group = group
        gname = group.group_name if hasattr(group, "group_name") else group
        self.partial = symm_mem.empty(max_tokens, hidden, dtype=torch.bfloat16, device=device)
        self.hbuf = symm_mem.empty(max_tokens, hidden, dtype=torch.bfloat16, device=device)
        self.sig_words = 8192  # one flag region; a second one serves the other half-batch of an overlapped step
        self.sig = symm_mem.empty(2 * self.sig_words, dtype=torch.int32, device=device)
        self.rows_cap = (max_tokens + size - 1) // size
        self.recv = symm_mem.empty(size * self.rows_cap, hidden, dtype=torch.bfloat16, device=device)
        self.agbuf = symm_mem.empty(self.rows_cap, hidden, dtype=torch.bfloat16, device=device)
        self.agflags = symm_mem.empty(1024, dtype=torch.int32, device=device)
        self.ag_staged = torch.empty(size * self.rows_cap, hidden, dtype=torch.bfloat16, device=device)
        # decode-sized steps: GEMM + word-flagged reduce-scatter + norm + gather in one kernel (gemm_ll_fused.cu)
        self.ll_max_tokens = int(os.environ.get("KSANA_LL_MAX_TOKENS", "256"))
        if hidden % 128 or hidden > 8192:
            self.ll_max_tokens = 0
        # two ranks: one hop (both ranks receive and reduce every row; the word buffer has two halves used in turn);
        # more ranks: reduce-scatter words to the row owners, then the owners' rows as words to everybody
        self.ll_one_shot = size == 2
        cap = max(self.ll_max_tokens, 1)
        self.ll_rows_cap = cap if self.ll_one_shot else (cap + size - 1) // size
        self.ll_half_words = size * self.ll_rows_cap * (hidden // 2)  # 8-byte words of one hop-1 buffer
        halves = 2 if self.ll_one_shot else 1
        self.ll_recv = symm_mem.empty(halves * self.ll_half_words * 2, dtype=torch.int32, device=device)
        self.ll_recv2 = symm_mem.empty(max(1 if self.ll_one_shot else cap * (hidden // 2), 64) * 2, dtype=torch.int32,
                                       device=device)
        self.ll_recv.zero_()
        self.ll_recv2.zero_()
        self.ll_seq = 0
        self.agbuf.zero_()
        self.agflags.zero_()
        self.recv.zero_()
        self.sig.zero_()
        self.partial.zero_()
        self.hbuf.zero_()
        torch.cuda.synchronize(device)
        self._h_partial = symm_mem.rendezvous(self.partial, gname)
        self._h_hbuf = symm_mem.rendezvous(self.hbuf, gname)
        self._h_sig = symm_mem.rendezvous(self.sig, gname)
        self._h_recv = symm_mem.rendezvous(self.recv, gname)
        self._h_agbuf = symm_mem.rendezvous(self.agbuf, gname)
        self._h_agflags = symm_mem.rendezvous(self.agflags, gname)
        self._h_ll_recv = symm_mem.rendezvous(self.ll_recv, gname)
        self._h_ll_recv2 = symm_mem.rendezvous(self.ll_recv2, gname)
        if use_multicast is None:
            use_multicast = os.environ.get("KSANA_DISABLE_MULTIMEM", "0") != "1"
        mc_ok = bool(use_multicast)
        self.partial_mc = int(self._h_partial.multicast_ptr) if mc_ok and self._h_partial.multicast_ptr else 0
        self.hbuf_mc = int(self._h_hbuf.multicast_ptr) if mc_ok and self._h_hbuf.multicast_ptr else 0
        if not (self.partial_mc and self.hbuf_mc):
            self.partial_mc = self.hbuf_mc = 0
        arr = ctypes.c_void_p * size
        self._partial_ptrs = arr(*[int(p) for p in self._h_partial.buffer_ptrs])
        self._hbuf_ptrs = arr(*[int(p) for p in self._h_hbuf.buffer_ptrs])
        self._sig_ptrs = arr(*[int(p) for p in self._h_sig.buffer_ptrs])
        self._recv_ptrs = arr(*[int(p) for p in self._h_recv.buffer_ptrs])
        self._agbuf_ptrs = arr(*[int(p) for p in self._h_agbuf.buffer_ptrs])
        self._agflag_ptrs = arr(*[int(p) for p in self._h_agflags.buffer_ptrs])
        self._ll_recv_ptrs = arr(*[int(p) for p in self._h_ll_recv.buffer_ptrs])
        self._ll_recv2_ptrs = arr(*[int(p) for p in self._h_ll_recv2.buffer_ptrs])
        self.ll_recv2_mc = int(self._h_ll_recv2.multicast_ptr) if mc_ok and self._h_ll_recv2.multicast_ptr else 0
        self.ag_epoch = 0
        self.single_kernel = os.environ.get("KSANA_DISABLE_FUSED_GEMM_RS", "0") != "1"
        self.comm_ctas = int(os.environ.get("KSANA_FUSED_COMM_CTAS", "16"))
        # Row-parallel GEMM + collective: ONE kernel (GEMM epilogue pushes tiles, communication warps reduce) or the
        # plain GEMM into symmetric memory followed by the reduce/norm/gather kernel. Measured (Llama-7B shapes,
        # 730 tokens): 2 ranks 1-kernel wins; 4 ranks 72 us vs 58 us and 8 ranks 81 us vs 48 us (64 tokens) for the
        # 2-kernel form at every size tried, so 4+ ranks always take it.
        self.two_kernel_max_tokens = int(os.environ.get("KSANA_TWO_KERNEL_MAX_TOKENS", "1048576" if size >= 4 else "0"))
        self.epoch = 0
        lib = kcuda.lib()
        lib.ksana_rs_norm_ag.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                         ctypes.c_uint, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.ksana_rs_norm_ag.restype = ctypes.c_int
        lib.ksana_gemm_rs_norm_ag.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float,
                                              ctypes.c_uint, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_void_p]
        lib.ksana_gemm_rs_norm_ag.restype = ctypes.c_int
        P, I = ctypes.c_void_p, ctypes.c_int
        LL = ctypes.c_longlong
        lib.ksana_gemm_ll_reduce_norm.argtypes = [P, P, I, I, I, I, I, I, I, P, LL, P, P, P, I, I, P, P, ctypes.c_float,
                                                  ctypes.c_uint, I, I, P]
        lib.ksana_gemm_ll_reduce_norm.restype = I
        lib.ksana_ll_reduce_norm.argtypes = [P, I, I, I, I, I, P, LL, P, P, P, I, I, P, P, ctypes.c_float, ctypes.c_uint,
                                             I, P]
        lib.ksana_ll_reduce_norm.restype = I
        lib.ksana_ag_wait_readers.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint,
                                              ctypes.c_void_p]
        lib.ksana_ag_wait_readers.restype = ctypes.c_int
        lib.ksana_gemm_allgather.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 7 + [
                                                 ctypes.c_uint, ctypes.c_void_p]
        lib.ksana_gemm_allgather.restype = ctypes.c_int
        self._lib = lib
        dist.barrier(group=group)
        # warm-up: lazy module loading and first-launch costs happen here, under a barrier, not inside a step
        z = torch.zeros(8, hidden, dtype=torch.bfloat16, device=device)
        self.all_reduce(z)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    @property
    def multicast(self) -> bool:
        return bool(self.partial_mc)

    # ---- capability checks used by TPGroup -----------------------------------------------------------------
    def can_all_reduce(self, x: torch.Tensor) -> bool:
        return (x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] == self.hidden and
                x.shape[0] <= self.max_tokens)

    def can_linear_reduce_norm(self, x: torch.Tensor, lin) -> bool:
        return x.dtype == torch.bfloat16 and lin.out_features == self.hidden and x.shape[0] <= self.max_tokens

    def next_epoch(self) -> int:
        """Epoch of the next collective on the shared buffers: grows by one per call, wraps modulo 2^32, never 0
        (0 is what untouched flag words hold)."""
        self.epoch += 1
        if self.epoch & 0xFFFFFFFF == 0:
            self.epoch += 1
        return self.epoch & 0xFFFFFFFF

    def _ll_recv_off(self) -> int:
        """Word offset of the hop-1 buffer half for the next small-step call (alternates with one hop)."""
        self.ll_seq += 1
        return (self.ll_seq & 1) * self.ll_half_words if self.ll_one_shot else 0

    # ---- kernels ------------------------------------------------------------------------------------------------
    def _launch_ll(self, y: torch.Tensor, residual, norm_w, eps: float) -> torch.Tensor:
        """Reduce (+ residual + norm) + gather of a partial sum in memory through the small-step kernel."""
        T = y.shape[0]
        if y.stride(1) != 1 or y.stride(0) % 4 or y.data_ptr() % 8:
            y = y.contiguous()
        mode = (1 if norm_w is not None else 0) | (2 if residual is not None else 0)
        code = self._lib.ksana_ll_reduce_norm(
            y.data_ptr(), y.stride(0), T, self.hidden, self.rank, self.size, self._ll_recv_ptrs, self._ll_recv_off(),
            self._ll_recv2_ptrs, self.ll_recv2_mc or None, self.hbuf.data_ptr(), self.ll_rows_cap,
            1 if self.ll_one_shot else 0, residual.data_ptr() if residual is not None else None,
            norm_w.data_ptr() if norm_w is not None else None, float(eps), self.next_epoch(), mode,
            torch.cuda.current_stream().cuda_stream)
        kcuda._check(code, "ll_reduce_norm")
        kcuda.launch_count += 1
        return self.hbuf[:T]

    def gemm_ll_reduce_add_norm(self, x, weight, residual, norm_w, eps) -> torch.Tensor:
        """Small steps: tcgen05 GEMM whose epilogue sends word-flagged slices to the row owners, which reduce,
        normalise and broadcast (csrc/cuda/gemm_ll_fused.cu)."""
        T, K = x.shape
        if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
            x = x.contiguous()
        mode = (1 if norm_w is not None else 0) | (2 if residual is not None else 0)
        code = self._lib.ksana_gemm_ll_reduce_norm(
            x.data_ptr(), weight.data_ptr(), T, self.hidden, K, x.stride(0), weight.stride(0), self.rank, self.size,
            self._ll_recv_ptrs, self._ll_recv_off(), self._ll_recv2_ptrs, self.ll_recv2_mc or None,
            self.hbuf.data_ptr(), self.ll_rows_cap, 1 if self.ll_one_shot else 0,
            residual.data_ptr() if residual is not None else None,
            norm_w.data_ptr() if norm_w is not None else None, float(eps), self.next_epoch(), mode, 0,
            torch.cuda.current_stream().cuda_stream)
        kcuda._check(code, "gemm_ll_reduce_norm")
        kcuda.launch_count += 1
        return self.hbuf[:T]

    def _launch(self, T: int, residual: Optional[torch.Tensor], norm_w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
        mode = (1 if norm_w is not None else 0) | (2 if residual is not None else 0)
        code = self._lib.ksana_rs_norm_ag(self.rank, self.size, self._partial_ptrs, self._hbuf_ptrs, self._sig_ptrs,
                                          self.partial_mc or None, self.hbuf_mc or None, T, self.hidden,
                                          residual.data_ptr() if residual is not None else None,
                                          norm_w.data_ptr() if norm_w is not None else None, float(eps),
                                          self.next_epoch(), mode, 0, torch.cuda.current_stream().cuda_stream)
        kcuda._check(code, "rs_norm_ag")
        return self.hbuf[:T]

    def linear_reduce_add_norm(self, x, lin, residual, norm_w, eps) -> torch.Tensor:
        """GEMM straight into the symmetric ``partial`` buffer, then the fused reduce/add/norm/gather kernel.
        The returned tensor is a view of ``hbuf`` (valid until the next fused call)."""
        T = x.shape[0]
        if (0 < T <= self.ll_max_tokens and lin.kind == "dense" and lin.bias is None and x.dim() == 2 and
                (residual is None or residual.is_contiguous())):
            return self.gemm_ll_reduce_add_norm(x, lin.weight, residual, norm_w, eps)
        if (self.single_kernel and T > self.two_kernel_max_tokens and lin.kind == "dense" and lin.bias is None and
                self.hidden % 256 == 0 and self.hidden <= 9216 and T <= 8192 and x.dim() == 2 and
                residual is not None and residual.is_contiguous()):
            return self.gemm_reduce_add_norm(x, lin.weight, residual, norm_w, eps)
        if lin.kind == "dense" and (lin.bias is None or self.rank != 0):
            kcuda.gemm_bf16(x, lin.weight, None, out=self.partial[:T])
        else:
            self.partial[:T].copy_(lin(x, add_bias=self.rank == 0))
        return self._launch(T, residual, norm_w, eps)

    def gemm_reduce_add_norm(self, x, weight, residual, norm_w, eps) -> torch.Tensor:
        """The single-kernel path: tcgen05 GEMM whose epilogue pushes tiles to the row owners over NVLink while
        communication CTAs reduce, normalise and broadcast finished row bands (csrc/cuda/gemm_fused_rs.cu)."""
        T, K = x.shape
        if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
            x = x.contiguous()
        mode = (1 if norm_w is not None else 0) | (2 if residual is not None else 0)
        code = self._lib.ksana_gemm_rs_norm_ag(
            x.data_ptr(), weight.data_ptr(), T, self.hidden, K, x.stride(0), weight.stride(0), self.rank, self.size,
            self._recv_ptrs, self._hbuf_ptrs, self._sig_ptrs, self.hbuf_mc or None, self.rows_cap,
            residual.data_ptr() if residual is not None else None,
            norm_w.data_ptr() if norm_w is not None else None, float(eps), self.next_epoch(), mode,
            self.comm_ctas, 0, torch.cuda.current_stream().cuda_stream)
        kcuda._check(code, "gemm_rs_norm_ag")
        return self.hbuf[:T]

    # ---- all-gather -> GEMM -------------------------------------------------------------------------------------
    def ag_rows(self, rows: int) -> torch.Tensor:
        """This rank's slice of the row-sharded activation ([rows, hidden] view of the symmetric buffer) for the next
        ``gemm_allgather``. The stream first waits until every peer has finished reading the previous contents."""
        assert rows <= self.rows_cap
        if self.ag_epoch:
            code = self._lib.ksana_ag_wait_readers(self.rank, self.size, self._agflag_ptrs,
                                                   self.ag_epoch & 0xFFFFFFFF, torch.cuda.current_stream().cuda_stream)
            kcuda._check(code, "ag_wait_readers")
        return self.agbuf[:rows]

    def gemm_allgather(self, rows_per: int, total_rows: int, weight: torch.Tensor,
                       bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """C[total_rows, N] = concat over ranks of their ``ag_rows(rows_per)`` contents times weight^T; every rank
        gets the full C. One kernel: A tiles are TMA-loaded from the owning rank's memory (csrc/cuda/
        gemm_allgather.cu)."""
        N = weight.shape[0]
        out = torch.empty(total_rows, N, dtype=torch.bfloat16, device=self.device)
        self.ag_epoch += 1
        code = self._lib.ksana_gemm_allgather(self.rank, self.size, self._agbuf_ptrs, self._agflag_ptrs,
                                              self.ag_staged.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                                              out.data_ptr(), rows_per, total_rows, N, self.hidden, self.hidden,
                                              weight.stride(0), N, self.ag_epoch & 0xFFFFFFFF,
                                              torch.cuda.current_stream().cuda_stream)
        kcuda._check(code, "gemm_allgather")
        kcuda.launch_count += 2
        return out

    def reduce_add_norm(self, y, residual, norm_w, eps) -> torch.Tensor:
        T = y.shape[0]
        if 0 < T <= self.ll_max_tokens and (residual is None or residual.is_contiguous()):
            return self._launch_ll(y, residual, norm_w, eps)
        self.partial[:T].copy_(y)
        return self._launch(T, residual, norm_w, eps)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        if 0 < T <= self.ll_max_tokens:
            return self._launch_ll(x, None, None, 0.0).clone()
        self.partial[:T].copy_(x)
        out = self._launch(T, None, None, 0.0)
        return out.clone()
