"""Fused compute + collective path over NVLink peer memory (the product; NCCL is the baseline).

``FusedComm`` owns this rank's symmetric receive buffers (``torch.distributed._symmetric_memory``
gives every rank a device pointer to every peer's copy) and routes the row-parallel projections
(attn_output, ffn_down) to ``oxb_gemm_ar``: one sm_100a kernel whose tcgen05 GEMM epilogue exchanges
each finished tile with the peers through P2P stores into their symmetric buffers and reduces the
partials as they arrive (decode batches: the whole grid is resident; prefill chunks: tile by tile,
overlapping the MMAs of the tiles behind).  Everything the fused kernels cannot take (more tokens
than the buffers hold, quantized row-parallel weights, odd shapes) falls back to the unfused GEMM
followed by an NCCL all-reduce, i.e. to the baseline, never to a wrong answer.

The reference has no GPU collectives (its data plane is a TCP ring,
``oxidize-core/src/mesh/ring.rs:245-365``); this module is what replaces it on NVSwitch.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from .comm import TorchComm

AR_MAX_TOKENS = 4096  # hard limit of the receive buffers (8 bytes x hidden x 2 x (W+1) per token row)
# Calls with more tokens than this go to GEMM + NCCL by default: the two-shot wire format carries an epoch beside
# every 4 bytes of payload, which wins on latency for decode batches and loses on bandwidth for prefill chunks.
FUSED_MAX_TOKENS = 256


class FusedComm(TorchComm):
    def __init__(self, device: torch.device, max_tokens: int = 256, hidden: int = 8192, group=None,
                 timeout_s: float = 5.0, max_tiles: int = 320, fused_max_tokens: int = FUSED_MAX_TOKENS):
        super().__init__(group)
        self.device = torch.device(device)
        self.t_max = max(16, min(int(max_tokens), int(fused_max_tokens), AR_MAX_TOKENS))
        self.n_max = int(hidden)
        self.max_tiles = int(max_tiles)
        self.timeout_ns = int(timeout_s * 1e9)
        self.fused_calls = 0
        self.fallback_calls = 0
        self.argmax_rows = 0
        W = self.size
        if W > 8:
            raise ValueError("fused collectives support up to 8 ranks (one NVSwitch domain)")
        self._handles = []
        if W > 1:
            import torch.distributed._symmetric_memory as symm

            pg = group if group is not None else dist.group.WORLD
            enable = getattr(symm, "enable_symm_mem_for_group", None)
            if enable is not None:
                try:
                    enable(pg.group_name)
                except Exception:
                    pass
            # 4 bytes per element: the LL exchange carries a 4-byte epoch beside every 4 bytes of payload
            self.data = symm.empty(2 * (W + 1) * self.t_max * self.n_max * 2, dtype=torch.bfloat16, device=self.device)
            self.flags = symm.empty(2 * (W + 1) * self.max_tiles, dtype=torch.int32, device=self.device)
            self.data.zero_()
            self.flags.zero_()
            h_data = symm.rendezvous(self.data, pg)
            h_flags = symm.rendezvous(self.flags, pg)
            # (value, index) pairs of the vocabulary-parallel argmax: [2 parities][W][rows][2] u64
            self.argmax_rows = 512
            self.amax = symm.empty(2 * W * self.argmax_rows * 2, dtype=torch.int64, device=self.device)
            self.amax.zero_()
            h_amax = symm.rendezvous(self.amax, pg)
            self._handles = [h_data, h_flags, h_amax]
            data_ptrs = [int(p) for p in h_data.buffer_ptrs]
            flag_ptrs = [int(p) for p in h_flags.buffer_ptrs]
            self._amax_ptrs = (ctypes.c_uint64 * 8)(*([int(p) for p in h_amax.buffer_ptrs] + [0] * (8 - W)))
            self.amax_ctrl = torch.zeros(4, dtype=torch.int32, device=self.device)
        else:
            self.data = torch.zeros(2 * 9 * self.t_max * self.n_max * 2, dtype=torch.bfloat16, device=self.device)
            self.flags = torch.zeros(2 * 9 * self.max_tiles, dtype=torch.int32, device=self.device)
            data_ptrs, flag_ptrs = [self.data.data_ptr()], [self.flags.data_ptr()]
        self.set_peer_pointers(data_ptrs, flag_ptrs)
        self.ctrl = torch.zeros(4, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self.barrier()

    def close(self) -> None:
        """Orderly end of the peer mappings: every rank stops launching, meets at a barrier (no kernel of a peer may
        still be writing into this rank's buffers) and only then drops its symmetric-memory handles and buffers."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.barrier()
        self._handles = []
        self.data = self.flags = None
        if hasattr(self, "amax"):
            self.amax = None

    def set_peer_pointers(self, data_ptrs, flag_ptrs, world: Optional[int] = None, rank: Optional[int] = None) -> None:
        """Install the peer pointer tables (also used by tests that emulate an absent peer)."""
        if world is not None:
            self.size = world
        if rank is not None:
            self.rank = rank
        self._data_ptrs = (ctypes.c_uint64 * 8)(*(list(data_ptrs) + [0] * (8 - len(data_ptrs))))
        self._flag_ptrs = (ctypes.c_uint64 * 8)(*(list(flag_ptrs) + [0] * (8 - len(flag_ptrs))))

    def argmax_exchange(self, logits: torch.Tensor, index_offset: int, tie: str = "lowest", feed=None) -> torch.Tensor:
        """Vocabulary-parallel greedy sampling in one kernel (see ``ops.cuda.argmax_tp``)."""
        from ..ops import cuda as C

        return C.argmax_tp(logits, tie, index_offset, self, feed)

    # ------------------------------------------------------------------ fused row-parallel linear
    def _fusable(self, x: torch.Tensor, w) -> bool:
        parts = getattr(w, "parts", [w])
        if not x.is_cuda or len(parts) != 1 or parts[0].qtype != "BF16" or getattr(w, "bias", None) is not None:
            return False
        T, K = x.shape
        N = parts[0].shape[0]
        if not (0 < T <= self.t_max and N <= self.n_max and N % 8 == 0 and K % 8 == 0):
            return False
        from ..ops import cuda as C

        return (N + 127) // 128 <= min(self.max_tiles, C.sm_count(x.device))

    def linear_allreduce(self, x: torch.Tensor, w, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """sum_r x_r @ W_r^T (+ residual) on every rank; fused when the shape allows."""
        if self.size == 1 or not self._fusable(x, w):
            self.fallback_calls += 1
            out = self.all_reduce(ops.linear(x, w))
            return out if residual is None else out + residual
        from ..ops import cuda as C

        part = getattr(w, "parts", [w])[0]
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = x.contiguous()
        T, K = x.shape
        N = part.shape[0]
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        s = C.scratch(x.device)
        C._check(C.lib().oxb_gemm_ar(x.data_ptr(), part.data.data_ptr(), out.data_ptr(), C._p(residual), T, N, K, N,
                                     self.size, self.rank, self._data_ptrs, self._flag_ptrs, self.ctrl.data_ptr(),
                                     self.t_max, self.n_max, self.max_tiles, ctypes.c_ulonglong(self.timeout_ns),
                                     s.gemm_ws.data_ptr(), s.gemm_ws.numel() * 4, s.gemm_counters.data_ptr(),
                                     s.gemm_counters.numel(), C._stream()), "oxb_gemm_ar")
        self.fused_calls += 1
        return out

    def linear_allreduce_into(self, x: torch.Tensor, w, residual: torch.Tensor, sumsq_out: torch.Tensor) -> bool:
        """residual += sum_r x_r @ W_r^T in place, inside the fused kernel, whose exchange also adds the sums of squares
        of the updated rows to ``sumsq_out`` ([>= T] int64, cleared beforehand: the producer half of a folded RMSNorm).
        False when the call cannot take the fused two-shot path (the caller then uses the unfused route)."""
        from ..ops import cuda as C

        if self.size == 1 or not self._fusable(x, w) or self.size < C.lib().oxb_set_ar_ll_min_world(-1):
            return False
        part = getattr(w, "parts", [w])[0]
        N = part.shape[0]
        if not residual.is_contiguous() or residual.dtype != torch.bfloat16:
            return False
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        x = x.contiguous()
        T, K = x.shape
        s = C.scratch(x.device)
        C._check(C.lib().oxb_gemm_ar_norm(x.data_ptr(), part.data.data_ptr(), residual.data_ptr(), residual.data_ptr(), T, N,
                                          K, N, self.size, self.rank, self._data_ptrs, self._flag_ptrs, self.ctrl.data_ptr(),
                                          self.t_max, self.n_max, self.max_tiles, ctypes.c_ulonglong(self.timeout_ns),
                                          s.gemm_ws.data_ptr(), s.gemm_ws.numel() * 4, s.gemm_counters.data_ptr(),
                                          s.gemm_counters.numel(), sumsq_out.data_ptr(), C._stream()), "oxb_gemm_ar_norm")
        self.fused_calls += 1
        return True

    # ------------------------------------------------------------------ stand-alone one-shot all-reduce
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if (self.size > 1 and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
                and 0 < x.shape[0] <= min(self.t_max, 512) and x.shape[1] <= self.n_max and x.shape[1] % 8 == 0
                and (x.shape[1] + 127) // 128 <= min(self.max_tiles, 148)):
            from ..ops import cuda as C

            T, N = x.shape
            C._check(C.lib().oxb_allreduce_oneshot(x.data_ptr(), x.data_ptr(), T, N, x.stride(0), self.size, self.rank,
                                                   self._data_ptrs, self._flag_ptrs, self.ctrl.data_ptr(), self.t_max,
                                                   self.n_max, self.max_tiles, ctypes.c_ulonglong(self.timeout_ns),
                                                   C._stream()), "oxb_allreduce_oneshot")
            self.fused_calls += 1
            return x
        return super().all_reduce(x)
