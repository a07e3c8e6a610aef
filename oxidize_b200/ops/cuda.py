"""ctypes bindings to ``liboxb.so`` (the hand-written sm_100a kernels) operating on torch CUDA
tensors.  Every function launches on the current torch stream, so the calls are captured by
``torch.cuda.graph`` like any other kernel.  Nothing here falls back to PyTorch math: a missing
library raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
LIB_PATH = os.path.join(_CSRC, "liboxb.so")

_lib = None
_lock = threading.Lock()

QTYPE_CODE = {"F32": 0, "F16": 1, "BF16": 2, "Q8_0": 3, "Q4_0": 4, "Q4_K": 5, "Q5_K": 6, "Q6_K": 7, "NVFP4": 8}
KV_MODE = {"bf16": 0, "f16": 1, "q8": 2, "q4": 3, "f32": 4}

SUMSQ_STRIDE = 16  # int64 words between the sum-of-squares accumulators of neighbouring tokens (folded RMSNorm)

launch_count = 0  # kernels launched through this module (bench.py reports it)


class OxbError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    from ..build import build_kernels

                    build_kernels()
                _lib = ctypes.CDLL(LIB_PATH)
                _declare(_lib)
    return _lib


@dataclass
class KernelOptions:
    """Process-wide switches of the kernel library (``EngineConfig.kernel_options``; the defaults are the tuned path,
    the alternatives exist for A/B measurements)."""

    pdl: bool = True  # programmatic dependent launch: a kernel's set-up overlaps the tail of the one before it
    cluster_splitk: bool = True  # split-K partials meet in distributed shared memory instead of global scratch
    gemm_prefill_tn: int = 256  # token tile of prefill-sized GEMM calls: 128, 256, or 0 = by wave count
    gemv_max_tokens: int = 2  # packed-weight calls of at most this many tokens take the dp4a GEMV (0 = never)
    gemv_wide: bool = False  # ... also for wide, short matrices (K >= 2N), where the split-K tensor-core kernel is faster
    ar_ll_min_world: int = 2  # rank counts from which the fused all-reduce uses the two-shot exchange
    # Packed-weight calls with more tokens than this decode the matrix to a bf16 staging buffer once and run the bf16
    # GEMM on it (every token tile of the fused kernel decodes the weight tile again: past ~900 tokens decoding once
    # wins, 1.4x at 2304 tokens); 0 = always the fused kernel.
    mmq_max_tokens: int = 1024
    # Checked mode: the op layer's scratch buffers (split-K partials and tickets, split-KV partials, decode staging) sit
    # between canary bands that ``verify_guards()`` checks (``LLM.step`` does so after every step, the kernel tests
    # after every test).  Costs a device synchronisation per check: for debugging, not for serving.
    checked: bool = False


mmq_max_tokens = KernelOptions.mmq_max_tokens
checked = False
_checked_forced = False


def _apply_checked(on: bool) -> None:
    global checked
    if on != checked:
        checked = on
        _scratch.clear()  # scratch is re-created with (or without) guard bands on next use


def set_checked(on: bool) -> None:
    """Checked mode for the whole process whatever later ``configure`` calls say (test suites)."""
    global _checked_forced
    _checked_forced = bool(on)
    _apply_checked(_checked_forced)



def configure(opts: "KernelOptions") -> None:
    L = lib()
    L.oxb_set_pdl(1 if opts.pdl else 0)
    L.oxb_set_cluster_splitk(1 if opts.cluster_splitk else 0)
    L.oxb_set_gemm_prefill_tn(int(opts.gemm_prefill_tn))
    L.oxb_set_gemv_max_tokens(int(opts.gemv_max_tokens))
    L.oxb_set_gemv_wide(1 if opts.gemv_wide else 0)
    L.oxb_set_ar_ll_min_world(int(opts.ar_ll_min_world))
    global mmq_max_tokens, checked
    mmq_max_tokens = int(opts.mmq_max_tokens)
    _apply_checked(bool(opts.checked) or _checked_forced)


def _declare(L) -> None:
    vp, i32, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    L.oxb_version.restype = i32
    L.oxb_status.argtypes = [ctypes.POINTER(i32), i32]
    L.oxb_gemm_plan.argtypes = [i32, i32, i32, i32, ctypes.POINTER(i32), ctypes.POINTER(sz), ctypes.POINTER(i32)]
    L.oxb_gemm_bf16.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, sz, vp, i32, vp]
    L.oxb_dequant_rows.argtypes = [vp, i32, sz, i32, i32, vp, i32, vp]
    L.oxb_embed.argtypes = [vp, vp, i32, sz, i32, i32, f32, vp, i32, vp]
    L.oxb_add_rmsnorm.argtypes = [vp, vp, vp, vp, vp, i32, i32, f32, vp]
    L.oxb_silu_mul.argtypes = [vp, vp, i32, i32, vp]
    L.oxb_gelu_mul.argtypes = [vp, vp, i32, i32, vp]
    L.oxb_qk_rope_kvwrite.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, i32, i32, i32, vp, vp, vp, i32,
                                      i32, i32, vp]
    L.oxb_argmax.argtypes = [vp, i32, i32, i32, i32, vp, vp, i32, vp]
    L.oxb_paged_attention.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, f32,
                                      vp, vp, vp, i32, vp]
    L.oxb_sample.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp, i32, vp, vp]
    L.oxb_gemm_quant.argtypes =[vp, vp, i32, sz, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, sz, vp, i32, vp]
    u64p, ull = ctypes.POINTER(ctypes.c_uint64), ctypes.c_ulonglong
    L.oxb_gemm_ar.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, u64p, u64p, vp, i32, i32, i32, ull, vp, sz,
                              vp, i32, vp]
    L.oxb_allreduce_oneshot.argtypes = [vp, vp, i32, i32, i32, i32, i32, u64p, u64p, vp, i32, i32, i32, ull, vp]
    L.oxb_gemm_bf16_norm.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, sz, vp, i32, vp, i32, f32, vp, vp, vp]
    L.oxb_gemm_ar_norm.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, u64p, u64p, vp, i32, i32, i32, ull, vp, sz,
                                   vp, i32, vp, vp]
    L.oxb_gemm_qkv_rope.argtypes = [vp, vp, i32, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp]
    L.oxb_gemm_qkv_rope_norm.argtypes = [vp, vp, i32, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, i32, f32,
                                         vp, vp]
    L.oxb_row_sumsq.argtypes = [vp, i32, i32, i32, vp, vp, vp]
    L.oxb_set_gemv_max_tokens.argtypes = [i32]
    L.oxb_set_gemv_wide.argtypes = [i32]


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise OxbError(f"{what} failed with CUDA error {code}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def status(reset: bool = True) -> Tuple[int, int, int]:
    """(code, detail, count) of the device status word; code 0 means every bounded wait succeeded."""
    out = (ctypes.c_int * 4)()
    _check(lib().oxb_status(out, 1 if reset else 0), "oxb_status")
    return out[0], out[1], out[2]


# --------------------------------------------------------------------------- scratch
class Scratch:
    """Per-device scratch owned by the op layer: split-K partials + tickets, split-KV partials,
    and the bf16 staging used to decode block-quantized weights ahead of the tensor-core GEMM."""

    def __init__(self, device: torch.device):
        self.device = device
        self.guards = None
        if checked:
            from ..utils.guards import GuardedAllocator

            self.guards = GuardedAllocator()
        self.gemm_ws = self._new(16 << 20, torch.float32, "gemm split-K partials")  # 64 MB
        self.gemm_counters = self._new(8192, torch.int32, "gemm split-K tickets", zero=True)
        self.attn_o: Optional[torch.Tensor] = None
        self.attn_ml: Optional[torch.Tensor] = None
        self.attn_counters = self._new(65536, torch.int32, "attention split tickets", zero=True)
        self.dequant: Optional[torch.Tensor] = None
        self._cap_attn = None
        self._cap_dequant = None

    def _new(self, n: int, dtype: torch.dtype, name: str, zero: bool = False, old: Optional[torch.Tensor] = None):
        """A buffer of this scratch; between canary bands in checked mode (never while a stream is capturing)."""
        if self.guards is not None and not torch.cuda.is_current_stream_capturing():
            if old is not None:
                self.guards.forget(old)
            return self.guards.empty(n, dtype, self.device, name, zero)
        return (torch.zeros if zero else torch.empty)(n, dtype=dtype, device=self.device)

    # The two growable buffers below must never be handed to a CUDA graph: growing them later would
    # free memory that the captured kernels still point to.  While a stream is capturing, the buffers
    # come from the graph's own memory pool instead (allocated once per capture, shared by its layers);
    # the eager warm-up that precedes every capture resets that per-capture arena.
    def attn(self, o_floats: int, ml_floats: int):
        if torch.cuda.is_current_stream_capturing():
            a = self._cap_attn
            if a is None or a[0].numel() < o_floats or a[1].numel() < ml_floats:
                a = self._cap_attn = (torch.empty(max(o_floats, 1), dtype=torch.float32, device=self.device),
                                      torch.empty(max(ml_floats, 1), dtype=torch.float32, device=self.device))
            return a
        self._cap_attn = None
        if self.attn_o is None or self.attn_o.numel() < o_floats:
            self.attn_o = self._new(max(o_floats, 1), torch.float32, "attention split-KV partial outputs", old=self.attn_o)
        if self.attn_ml is None or self.attn_ml.numel() < ml_floats:
            self.attn_ml = self._new(max(ml_floats, 1), torch.float32, "attention split-KV max / sum", old=self.attn_ml)
        return self.attn_o, self.attn_ml

    def dequant_buf(self, n: int) -> torch.Tensor:
        if torch.cuda.is_current_stream_capturing():
            if self._cap_dequant is None or self._cap_dequant.numel() < n:
                self._cap_dequant = torch.empty(n, dtype=torch.bfloat16, device=self.device)
            return self._cap_dequant
        self._cap_dequant = None
        if self.dequant is None or self.dequant.numel() < n:
            self.dequant = self._new(n, torch.bfloat16, "packed-weight decode staging", old=self.dequant)
        return self.dequant


_scratch: Dict[int, Scratch] = {}


def scratch(device: torch.device) -> Scratch:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _scratch.get(idx)
    if s is None:
        s = _scratch[idx] = Scratch(torch.device("cuda", idx))
    return s


def verify_guards() -> None:
    """Checked mode: raise ``utils.guards.MemoryGuardError`` if a kernel wrote outside one of the scratch buffers
    (synchronises every device that has scratch).  Does nothing otherwise."""
    for s in _scratch.values():
        if s.guards is not None:
            torch.cuda.synchronize(s.device)
            s.guards.verify()


# --------------------------------------------------------------------------- GEMM / linear
def gemm_plan(T: int, N: int, K: int, splits_hint: int = 0):
    out = (ctypes.c_int * 4)()
    ws = ctypes.c_size_t()
    nc = ctypes.c_int()
    lib().oxb_gemm_plan(T, N, K, splits_hint, out, ctypes.byref(ws), ctypes.byref(nc))
    return {"tn": out[0], "n_tiles": out[1], "t_tiles": out[2], "splits": out[3], "ws_bytes": ws.value,
            "n_counters": nc.value}


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
              ld_out: Optional[int] = None, add_into: bool = False, splits: int = 0, swiglu: bool = False,
              sumsq_in: Optional[torch.Tensor] = None, eps: float = 0.0, clear: Optional[torch.Tensor] = None,
              sumsq_out: Optional[torch.Tensor] = None, gelu: bool = False) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w[N, K]^T on the tcgen05 kernel; ``out`` may be a column slice of a
    wider row-major buffer (pass its row stride as ``ld_out``).

    The three accumulator arguments (int64 tensors of 2^-28 fixed-point sums of squares, token t at word
    ``t * SUMSQ_STRIDE``, see :func:`row_sumsq`)
    make the call one half of a folded RMSNorm.  ``sumsq_in``: ``x`` holds un-normalised rows and token t's result is
    scaled by 1/rms(x_t); ``clear`` is zeroed on the way for the producer that follows.  ``sumsq_out``: the epilogue adds
    the sums of squares of the rows it writes (the producer half; the array must have been cleared)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty(T, N // 2 if swiglu else N, dtype=torch.bfloat16, device=x.device)
        ld_out = out.stride(0)
    elif ld_out is None:
        ld_out = out.stride(0)
    s = scratch(x.device)
    epi = (4 if gelu else 2) if swiglu else (1 if add_into else 0)  # EPI_GEGLU / EPI_SWIGLU / EPI_ADD_INTO / EPI_STORE
    if sumsq_in is None and sumsq_out is None:
        _check(lib().oxb_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), _p(bias), T, N, K, ld_out, epi, splits,
                                   s.gemm_ws.data_ptr(), s.gemm_ws.numel() * 4, s.gemm_counters.data_ptr(),
                                   s.gemm_counters.numel(), _stream()), "oxb_gemm_bf16")
        return out
    _check(lib().oxb_gemm_bf16_norm(x.data_ptr(), w.data_ptr(), out.data_ptr(), _p(bias), T, N, K, ld_out, epi, splits,
                                    s.gemm_ws.data_ptr(), s.gemm_ws.numel() * 4, s.gemm_counters.data_ptr(),
                                    s.gemm_counters.numel(), _p(sumsq_in), K, eps, _p(clear), _p(sumsq_out), _stream()),
           "oxb_gemm_bf16_norm")
    return out


def row_sumsq(x: torch.Tensor, out: torch.Tensor, clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t * SUMSQ_STRIDE] (int64, 2^-28 fixed point) = sum of squares of row t of ``x`` (bf16 [T, H]); the same
    words of ``clear`` are zeroed."""
    T, H = x.shape
    _check(lib().oxb_row_sumsq(x.data_ptr(), x.stride(0), T, H, out.data_ptr(), _p(clear), _stream()), "oxb_row_sumsq")
    return out


class l2_prefetch:
    """``with l2_prefetch(kb):`` GEMMs launched inside request up to ``kb`` weight k-blocks (16 KB each) per
    CTA into the L2 before their grid dependency resolves.  Worth it only behind a collective, whose
    wait leaves HBM idle; behind an HBM-bound kernel it costs 10-20%."""

    def __init__(self, kb: int):
        self.kb = int(kb)

    def __enter__(self):
        self.old = lib().oxb_set_gemm_l2_prefetch(self.kb) if self.kb > 0 else 0
        return self

    def __exit__(self, *exc):
        if self.kb > 0:
            lib().oxb_set_gemm_l2_prefetch(self.old)
        return False


def dequant_rows(w, out: Optional[torch.Tensor] = None, fast: bool = False) -> torch.Tensor:
    """Decode a packed QTensor to a dense bf16 [out, in] matrix on the device.  ``fast`` uses the vectorised decoder of
    the fused GEMM where it applies (Q4_K / Q6_K / Q8_0; block scales rounded to bf16), else the exact one."""
    n, k = w.shape
    if out is None:
        out = torch.empty(n, k, dtype=torch.bfloat16, device=w.data.device)
    _check(lib().oxb_dequant_rows(w.data.data_ptr(), QTYPE_CODE[w.qtype], w.data.stride(0) * w.data.element_size(), n, k,
                                  out.data_ptr(), 1 if fast else 0, _stream()), "oxb_dequant_rows")
    return out


def linear(x: torch.Tensor, parts: Sequence, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    x = x.contiguous()
    T = x.shape[0]
    N = sum(p.shape[0] for p in parts)
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    off = 0
    for p in parts:
        n = p.shape[0]
        b = None if bias is None else bias[off : off + n]
        view = out[:, off : off + n]
        if p.qtype == "BF16":
            gemm_bf16(x, p.data, view, b, ld_out=out.stride(0))
        elif p.qtype in ("F32", "F16"):
            if getattr(p, "_bf16", None) is None:
                p._bf16 = p.data.to(torch.bfloat16).contiguous()
            gemm_bf16(x, p._bf16, view, b, ld_out=out.stride(0))
        elif p.qtype == "FP8B":
            from . import cuda_quant

            cuda_quant.linear_fp8(x, p, view, b, out.stride(0))
        else:
            from . import cuda_quant

            cuda_quant.linear_quant(x, p, view, b, out.stride(0))
        off += n
    return out


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[gate (F rows); up (F rows)] -> per 128-row tile: 64 gate rows followed by their 64 up rows
    (the layout the GEMM's SwiGLU epilogue expects).  F must be a multiple of 64."""
    F = w.shape[0] // 2
    g = w[:F].reshape(F // 64, 64, -1)
    u = w[F:].reshape(F // 64, 64, -1)
    return torch.cat([g, u], dim=1).reshape(2 * F, -1).contiguous()


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, sumsq_in: Optional[torch.Tensor] = None,
                  eps: float = 0.0, clear: Optional[torch.Tensor] = None, gelu: bool = False) -> torch.Tensor:
    """act(x W_gate^T) * (x W_up^T) in ONE kernel: the activation (SiLU, or tanh-GELU with ``gelu``) is the GEMM's
    epilogue."""
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    return gemm_bf16(x.contiguous(), w_interleaved, swiglu=True, sumsq_in=sumsq_in, eps=eps, clear=clear, gelu=gelu)


# --------------------------------------------------------------------------- glue ops
def embed(tokens: torch.Tensor, table, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    T = tokens.shape[0]
    V, H = table.shape
    out = torch.empty(T, H, dtype=torch.bfloat16, device=tokens.device)
    row_bytes = table.data.stride(0) * table.data.element_size()
    _check(lib().oxb_embed(tokens.data_ptr(), table.data.data_ptr(), QTYPE_CODE[table.qtype], row_bytes, H, V, scale,
                           out.data_ptr(), T, _stream()), "oxb_embed")
    return out if dtype == torch.bfloat16 else out.to(dtype)


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], w: torch.Tensor, eps: float):
    """(rmsnorm(x + residual) * w, x + residual); the sum overwrites ``residual`` in place."""
    T, H = x.shape
    y = torch.empty_like(x)
    if residual is None:
        _check(lib().oxb_add_rmsnorm(x.data_ptr(), None, None, w.data_ptr(), y.data_ptr(), T, H, eps, _stream()),
               "oxb_add_rmsnorm")
        return y, x
    _check(lib().oxb_add_rmsnorm(x.data_ptr(), residual.data_ptr(), residual.data_ptr(), w.data_ptr(), y.data_ptr(),
                                 T, H, eps, _stream()), "oxb_add_rmsnorm")
    return y, residual


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    T, I2 = gate_up.shape
    out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().oxb_silu_mul(gate_up.data_ptr(), out.data_ptr(), T, I2 // 2, _stream()), "oxb_silu_mul")
    return out


def gelu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """tanh-GELU(gate) * up (GeGLU) on a fused bf16 [T, 2F] projection."""
    T, I2 = gate_up.shape
    out = torch.empty(T, I2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().oxb_gelu_mul(gate_up.data_ptr(), out.data_ptr(), T, I2 // 2, _stream()), "oxb_gelu_mul")
    return out


def rope_table(rope, max_pos: int) -> torch.Tensor:
    """[max_pos, rot] fp32: cos at [:, :rot/2], sin at [:, rot/2:], computed in float64."""
    tab = getattr(rope, "_table", None)
    if tab is None or tab.shape[0] < max_pos:
        n = max(max_pos, 32768)
        pos = torch.arange(n, dtype=torch.float64, device=rope.inv_freq.device)
        ang = pos[:, None] * rope.inv_freq.double()[None, :]
        tab = torch.cat([ang.cos() * rope.mscale, ang.sin() * rope.mscale], dim=1).float().contiguous()
        rope._table = tab
    return tab


def qk_rope_kv_write(qkv, positions, slot_mapping, kv, layer, rope, q_norm=None, k_norm=None, eps=1e-6):
    T = qkv.shape[0]
    nq, nkv, hd = rope.n_heads, rope.n_kv_heads, rope.head_dim
    tab = rope_table(rope, 0)
    q = torch.empty(T, nq, hd, dtype=torch.bfloat16, device=qkv.device)
    rot = tab.shape[1]
    sc = kv.scales[layer]
    _check(lib().oxb_qk_rope_kvwrite(qkv.data_ptr(), positions.data_ptr(), slot_mapping.data_ptr(), tab.data_ptr(),
                                     tab.shape[0], rot, 0 if rope.pairing == "split_half" else 1, _p(q_norm),
                                     _p(k_norm), eps, T, nq, nkv, hd, q.data_ptr(), kv.data[layer].data_ptr(), _p(sc),
                                     KV_MODE[kv.dtype_name], kv.page_size, kv.num_blocks, _stream()), "oxb_qk_rope_kvwrite")
    return q


def qkv_rope_fusable(w_parts, kv, rope, q_norm, k_norm) -> bool:
    """The fused qkv GEMM + RoPE + KV-write kernel covers the common case: one bf16 weight, head_dim 128,
    full rotary, no QK-norm, bf16 KV pages."""
    return (len(w_parts) == 1 and w_parts[0].qtype == "BF16" and rope.head_dim == 128 and q_norm is None
            and k_norm is None and kv.dtype_name == "bf16" and rope_table(rope, 0).shape[1] == 128
            and w_parts[0].shape[0] == (rope.n_heads + 2 * rope.n_kv_heads) * 128)


def linear_qkv_rope(x: torch.Tensor, w: torch.Tensor, positions, slot_mapping, kv, layer, rope,
                    sumsq_in: Optional[torch.Tensor] = None, eps: float = 0.0,
                    clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q = RoPE(x Wq^T) as [T, nq, 128]; RoPE(x Wk^T) and x Wv^T go straight into the paged KV cache:
    one kernel instead of the qkv GEMM followed by the RoPE / KV-write kernel.  With ``sumsq_in`` the rows of
    ``x`` are un-normalised and the kernel applies 1/rms per token (folded RMSNorm, see :func:`gemm_bf16`)."""
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    x = x.contiguous()
    T, K = x.shape
    nq, nkv = rope.n_heads, rope.n_kv_heads
    tab = rope_table(rope, 0)
    q = torch.empty(T, nq, 128, dtype=torch.bfloat16, device=x.device)
    L = lib()
    pairing = 0 if rope.pairing == "split_half" else 1
    if sumsq_in is None:
        _check(L.oxb_gemm_qkv_rope(x.data_ptr(), w.data_ptr(), T, K, positions.data_ptr(), slot_mapping.data_ptr(),
                                   tab.data_ptr(), tab.shape[0], tab.shape[1], pairing, nq, nkv, q.data_ptr(),
                                   kv.data[layer].data_ptr(), kv.page_size, kv.num_blocks, _stream()), "oxb_gemm_qkv_rope")
    else:
        _check(L.oxb_gemm_qkv_rope_norm(x.data_ptr(), w.data_ptr(), T, K, positions.data_ptr(), slot_mapping.data_ptr(),
                                        tab.data_ptr(), tab.shape[0], tab.shape[1], pairing, nq, nkv, q.data_ptr(),
                                        kv.data[layer].data_ptr(), kv.page_size, kv.num_blocks, sumsq_in.data_ptr(), K, eps,
                                        _p(clear), _stream()), "oxb_gemm_qkv_rope_norm")
    return q


_SM_COUNT: Dict[int, int] = {}


def sm_count(device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def attn_splits(B: int, nkv: int, mtiles: int, max_seq_len: int, sms: int) -> int:
    """CTA-level KV splits: as many as keep the grid within ONE wave of two CTAs per SM (a partly
    filled second wave doubles the kernel's time) while each warp of each split still sees a few
    pages."""
    base = max(1, B * nkv * mtiles)
    want = max(1, (2 * sms) // base)
    pages = max(1, (max_seq_len + 15) // 16)
    cap = max(1, pages // 8)  # >= 2 pages per warp per split
    return max(1, min(want, cap, 16))


def paged_attention(q, kv, layer, meta, scale, sliding_window=0, splits: Optional[int] = None, softcap: float = 0.0):
    T, nq, hd = q.shape
    nkv = kv.spec.n_kv_heads
    B = meta.seq_lens.shape[0]
    G = nq // nkv
    mtiles = (max(1, meta.max_query_len) * G + 15) // 16
    if splits is None:
        splits = attn_splits(B, nkv, mtiles, meta.max_seq_len or kv.page_size, sm_count(q.device))
    out = torch.empty_like(q)
    ws_o = ws_ml = cnt = None
    if splits > 1 and B * nkv * mtiles > scratch(q.device).attn_counters.numel():
        splits = 1
    if splits > 1:
        tasks = B * nkv * mtiles * splits
        ws_o, ws_ml = scratch(q.device).attn(tasks * 16 * hd, tasks * 32)
        cnt = scratch(q.device).attn_counters
    _check(lib().oxb_paged_attention(q.data_ptr(), out.data_ptr(), kv.data[layer].data_ptr(), _p(kv.scales[layer]),
                                     meta.block_tables.data_ptr(), meta.seq_lens.data_ptr(), meta.query_start.data_ptr(),
                                     B, meta.block_tables.stride(0), nq, nkv, hd, KV_MODE[kv.dtype_name],
                                     max(1, meta.max_query_len), splits, sliding_window, scale, float(softcap), _p(ws_o),
                                     _p(ws_ml),
                                     _p(cnt), kv.num_blocks, _stream()), "oxb_paged_attention")
    return out


def argmax(logits: torch.Tensor, tie: str = "lowest", out_val: Optional[torch.Tensor] = None, index_offset: int = 0):
    assert logits.dtype == torch.float32
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    _check(lib().oxb_argmax(logits.data_ptr(), R, V, logits.stride(0), 1 if tie == "highest" else 0, out.data_ptr(),
                            _p(out_val), index_offset, _stream()), "oxb_argmax")
    return out


def argmax_tp(logits: torch.Tensor, tie: str = "lowest", index_offset: int = 0, comm=None,
              feed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row from this rank's logits shard (fp32 or bf16); with ``comm`` (a FusedComm) the
    (value, index) pairs of all tensor-parallel ranks are exchanged inside the kernel.  ``feed`` also receives the tokens."""
    R, V = logits.shape
    dt = {torch.float32: 0, torch.bfloat16: 2}[logits.dtype]
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    L = lib()
    if not getattr(L, "_argmax_tp_declared", False):
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        L.oxb_argmax_tp.argtypes = [vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, i32, ctypes.POINTER(ctypes.c_uint64), vp, i32,
                                    ctypes.c_ulonglong, vp]
        L._argmax_tp_declared = True
    if comm is None:
        _check(L.oxb_argmax_tp(logits.data_ptr(), dt, R, V, logits.stride(0), 1 if tie == "highest" else 0, out.data_ptr(),
                               _p(feed), index_offset, 1, 0, None, None, 0, 0, _stream()), "oxb_argmax_tp")
    else:
        _check(L.oxb_argmax_tp(logits.data_ptr(), dt, R, V, logits.stride(0), 1 if tie == "highest" else 0, out.data_ptr(),
                               _p(feed), index_offset, comm.size, comm.rank, comm._amax_ptrs, comm.amax_ctrl.data_ptr(),
                               comm.argmax_rows, ctypes.c_ulonglong(comm.timeout_ns), _stream()), "oxb_argmax_tp")
    return out


def spec_verify(target_logits: torch.Tensor, draft_logits: Optional[torch.Tensor], draft_tokens: torch.Tensor,
                row0: torch.Tensor, n_draft: torch.Tensor, temperature: torch.Tensor, uniforms: torch.Tensor, K: int,
                tie: str = "lowest"):
    """Verify the K drafted tokens of each of S sequences against their K+1 rows of target logits in one launch.
    Returns (tokens [S, K+1] int32, count [S] int32): count[s] tokens were emitted for sequence s.  Greedy rows
    (temperature <= 0) use the exact-match rule, sampled rows min(1, p/q) acceptance with residual resampling."""
    S = int(row0.shape[0])
    V = int(target_logits.shape[1])
    assert target_logits.dtype == torch.float32 and (draft_logits is None or draft_logits.dtype == torch.float32)
    toks = torch.zeros(S, K + 1, dtype=torch.int32, device=target_logits.device)
    cnt = torch.zeros(S, dtype=torch.int32, device=target_logits.device)
    L = lib()
    if not getattr(L, "_spec_verify_declared", False):
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        L.oxb_spec_verify.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
        L._spec_verify_declared = True
    _check(L.oxb_spec_verify(target_logits.data_ptr(), target_logits.stride(0), _p(draft_logits),
                             0 if draft_logits is None else draft_logits.stride(0), draft_tokens.data_ptr(), row0.data_ptr(),
                             n_draft.data_ptr(), temperature.data_ptr(), uniforms.data_ptr(), toks.data_ptr(), cnt.data_ptr(),
                             S, K, V, 1 if tie == "highest" else 0, _stream()), "oxb_spec_verify")
    return toks, cnt


def sample(logits, temperature, top_k, top_p, min_p, random, tie="lowest"):
    from . import cuda_sampling

    return cuda_sampling.sample(logits, temperature, top_k, top_p, min_p, random, tie)


def moe_route(logits, cfg, bias=None):
    from . import cuda_moe

    return cuda_moe.moe_route(logits, cfg, bias)


def moe_experts_forward(x, ids, wts, experts):
    from . import cuda_moe

    return cuda_moe.moe_experts_forward(x, ids, wts, experts)
