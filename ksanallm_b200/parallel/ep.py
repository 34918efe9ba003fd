"""Expert-parallel dispatch / combine over NVLink peer memory (csrc/cuda/moe_ep.cu).

Each rank owns a slice of the step's tokens and a slice of the experts. ``EPExchange.moe`` sends every token row once
to each rank that hosts one of its experts, runs the local sort + grouped-GEMM pipeline on what arrived, and returns
the weighted expert outputs of the rank's own tokens. The reference reaches the same result either with DeepEP in a
helper process (src/ksana_llm/data_hub/expert_parallel_deepep_wrapper.cpp:31-330) or, inside one node, by replicating
all tokens on all ranks and all-reducing the outputs (src/ksana_llm/layers/nvidia/moe_layer.cpp ExpertMap path).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import cuda as kcuda
from ..ops import cuda_moe


def _align(n: int, a: int = 1024) -> int:
    return (n + a - 1) // a * a


class EPExchange:
    def __init__(self, group, rank: int, size: int, device: torch.device, hidden: int, top_k: int, num_experts: int,
                 max_tokens_per_rank: int):
        import torch.distributed._symmetric_memory as symm_mem
        assert num_experts % size == 0 and size <= 8
        self.rank, self.size, self.device, self.group = rank, size, device, group
        self.hidden, self.top_k = hidden, top_k
        self.e_local = num_experts // size
        self.t_cap = max_tokens_per_rank
        rows = size * max_tokens_per_rank
        self._row_bytes = rows * hidden * 2
        self._meta_bytes = rows * top_k * 4
        total = 2 * _align(self._row_bytes) + 2 * _align(self._meta_bytes) + 1024
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        gname = group.group_name if hasattr(group, "group_name") else group
        self._handle = symm_mem.rendezvous(self.buf, gname)
        self._ptrs = (ctypes.c_void_p * size)(*[int(p) for p in self._handle.buffer_ptrs])
        self.epoch = 0
        self.step_stride = 0  # attention-DP mode: slot stride of the current step (set by the engine)
        lib = kcuda.lib()
        P, I, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint
        lib.ksana_ep_dispatch.argtypes = [I, I, P, P, P, I, P, P, I, I, I, I, I, U, P]
        lib.ksana_ep_combine.argtypes = [I, I, P, P, P, P, I, I, I, U, P]
        lib.ksana_ep_finish.argtypes = [I, I, P, P, P, I, I, I, I, I, P, I, P, I, U, P]
        for f in (lib.ksana_ep_dispatch, lib.ksana_ep_combine, lib.ksana_ep_finish):
            f.restype = I
        self._lib = lib
        dist.barrier(group=group)

    def _layout(self):
        """Byte offsets of the regions. They never move (only the slot stride inside a region changes from call to
        call), so a region is only ever written by one kind of kernel and the epoch flags order every reuse."""
        off_x = 0
        off_ret = _align(self._row_bytes)
        off_ids = 2 * _align(self._row_bytes)
        off_w = off_ids + _align(self._meta_bytes)
        off_flags = off_w + _align(self._meta_bytes)
        return (ctypes.c_longlong * 5)(off_x, off_ret, off_ids, off_w, off_flags), (off_x, off_ret, off_ids, off_w)

    def moe(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
            w_down: torch.Tensor, t_stride: int, add: Optional[torch.Tensor] = None, fp8_scales=None) -> torch.Tensor:
        """x [T_local, H] bf16 (this rank's tokens), ids / weights [T_local, k] with GLOBAL expert ids, expert
        weights of the rank's ``num_experts / size`` local experts. ``t_stride`` >= every rank's T_local and equal
        on all ranks. Returns [T_local, H] = add + sum_k w_k * expert_k(x).

        ``fp8_scales`` = (gate_up scales, down scales) of block-scaled e4m3 expert weights: the token rows are then
        quantised BEFORE they leave (e4m3 values + one fp32 scale per 128 channels: H + H / 32 bytes per row instead
        of 2 H), the receiving rank's grouped fp8 GEMM reads them in place, outputs return in bf16."""
        T, H = x.shape
        k = self.top_k
        assert t_stride <= self.t_cap and T <= t_stride and H == self.hidden and ids.shape[1] == k
        if fp8_scales is not None:
            return self._moe_fp8(x, ids, weights, w_gate_up, w_down, fp8_scales, t_stride, add)
        offs, (off_x, off_ret, off_ids, off_w) = self._layout()
        self.epoch += 1
        ep = self.epoch & 0xFFFFFFFF
        st = torch.cuda.current_stream().cuda_stream
        idc = ids.to(torch.int32).contiguous()
        wc = weights.float().contiguous()
        xc = x if x.stride(1) == 1 and x.stride(0) % 8 == 0 else x.contiguous()
        kcuda._check(self._lib.ksana_ep_dispatch(self.rank, self.size, self._ptrs, offs, xc.data_ptr() if T else None,
                                                 xc.stride(0) if T else H, idc.data_ptr() if T else None,
                                                 wc.data_ptr() if T else None, T, t_stride, k, H, self.e_local, ep,
                                                 st), "ep_dispatch")
        rows = self.size * t_stride
        recv_x = self.buf[off_x:off_x + rows * H * 2].view(torch.bfloat16).view(rows, H)
        recv_ids = self.buf[off_ids:off_ids + rows * k * 4].view(torch.int32).view(rows, k)
        y, pos = cuda_moe.expert_pipeline(recv_x, recv_ids, w_gate_up, w_down, self.rank * self.e_local)
        kcuda._check(self._lib.ksana_ep_combine(self.rank, self.size, self._ptrs, offs, y.data_ptr(), pos.data_ptr(),
                                                t_stride, k, H, ep, st), "ep_combine")
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        kcuda._check(self._lib.ksana_ep_finish(self.rank, self.size, self._ptrs, offs, idc.data_ptr() if T else None,
                                               T, t_stride, k, H, self.e_local,
                                               add.data_ptr() if add is not None else None,
                                               add.stride(0) if add is not None else 0, out.data_ptr() if T else None,
                                               H, ep, st), "ep_finish")
        kcuda.launch_count += 4
        return out

    def _moe_fp8(self, x, ids, weights, wq_gate_up, wq_down, scales, t_stride, add) -> torch.Tensor:
        T, H = x.shape
        k = self.top_k
        assert H % 512 == 0, "packed fp8 rows need H + H / 32 bytes to be a multiple of 16"
        hp = (H + H // 32) // 2  # packed row as bf16 elements (the dispatch kernel moves 16-byte pieces)
        offs, (off_x, off_ret, off_ids, off_w) = self._layout()
        self.epoch += 1
        ep = self.epoch & 0xFFFFFFFF
        st = torch.cuda.current_stream().cuda_stream
        idc = ids.to(torch.int32).contiguous()
        wc = weights.float().contiguous()
        packed = cuda_moe.pack_fp8_rows(x).view(torch.bfloat16) if T else x[:, :hp]
        kcuda._check(self._lib.ksana_ep_dispatch(self.rank, self.size, self._ptrs, offs,
                                                 packed.data_ptr() if T else None, hp, idc.data_ptr() if T else None,
                                                 wc.data_ptr() if T else None, T, t_stride, k, hp, self.e_local, ep,
                                                 st), "ep_dispatch")
        rows = self.size * t_stride
        recv_x = self.buf[off_x:off_x + rows * hp * 2].view(torch.bfloat16).view(rows, hp)
        recv_ids = self.buf[off_ids:off_ids + rows * k * 4].view(torch.int32).view(rows, k)
        y, pos = cuda_moe.expert_pipeline_fp8(recv_x, recv_ids, wq_gate_up, scales[0], wq_down, scales[1],
                                              self.rank * self.e_local, packed=True)
        kcuda._check(self._lib.ksana_ep_combine(self.rank, self.size, self._ptrs, offs, y.data_ptr(), pos.data_ptr(),
                                                t_stride, k, H, ep, st), "ep_combine")
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
        kcuda._check(self._lib.ksana_ep_finish(self.rank, self.size, self._ptrs, offs, idc.data_ptr() if T else None,
                                               T, t_stride, k, H, self.e_local,
                                               add.data_ptr() if add is not None else None,
                                               add.stride(0) if add is not None else 0, out.data_ptr() if T else None,
                                               H, ep, st), "ep_finish")
        kcuda.launch_count += 4
        return out
