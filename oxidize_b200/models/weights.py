"""Weight containers and the shard-aware GGUF loader.

Weights stay in their checkpoint encoding on the device (packed Q4_K / Q6_K / Q8_0 / NVFP4
rows, or bf16); a tensor-parallel rank copies only its slice of the mmap:

* column-parallel (q, k, v, gate, up, experts' gate/up, lm_head): a contiguous range of rows;
* row-parallel (attn_output, ffn_down): a contiguous range of *columns*, cut on quant-block
  boundaries (256 for k-quants), i.e. a byte range inside every row.

Tensor names are the GGUF ones the reference maps at ``model/inference/load.rs:81-431``;
``output.weight`` absent means the head is tied to the embedding (``load.rs:436``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..formats.gguf import GGUFFile, GGMLTypeInfo, ggml_type
from ..quant import ref as qref
from .config import ModelConfig


@dataclass
class QTensor:
    """A 2-D weight ``[out, in]`` in its storage encoding.

    ``data`` is ``[out, in]`` for F32/F16/BF16 and ``uint8 [out, row_bytes]`` for block
    formats.  ``FP8B`` is our block-scaled fp8 (e4m3 codes + one f32 scale per ``block``
    input channels), which has no GGUF id."""

    qtype: str
    data: torch.Tensor
    shape: Tuple[int, int]
    scales: Optional[torch.Tensor] = None
    block: int = 128
    _dense: Optional[torch.Tensor] = field(default=None, repr=False)

    @property
    def out_features(self) -> int:
        return self.shape[0]

    @property
    def in_features(self) -> int:
        return self.shape[1]

    @property
    def device(self):
        return self.data.device

    def nbytes(self) -> int:
        n = self.data.numel() * self.data.element_size()
        if self.scales is not None:
            n += self.scales.numel() * self.scales.element_size()
        return n

    def dense_cache(self) -> torch.Tensor:
        """float32 dense copy, decoded once (CPU reference path / tests only)."""
        if self._dense is None:
            from ..ops import ref as opref

            self._dense = opref.dequantize_weight(self)
        return self._dense

    def to(self, device) -> "QTensor":
        return QTensor(self.qtype, self.data.to(device), self.shape,
                       None if self.scales is None else self.scales.to(device), self.block)

    def rows(self, start: int, stop: int) -> "QTensor":
        return QTensor(self.qtype, self.data[start:stop], (stop - start, self.shape[1]),
                       None if self.scales is None else self.scales[start:stop], self.block)


def qtensor_from_dense(w: torch.Tensor, qtype: str = "BF16", device=None) -> QTensor:
    """Encode a dense float weight ``[out, in]`` into ``qtype`` (host-side, NumPy oracle)."""
    qtype = qtype.upper()
    out_f, in_f = w.shape
    dev = device if device is not None else w.device
    if qtype == "F32":
        return QTensor("F32", w.float().to(dev).contiguous(), (out_f, in_f))
    if qtype == "BF16":
        return QTensor("BF16", w.to(torch.bfloat16).to(dev).contiguous(), (out_f, in_f))
    if qtype == "F16":
        return QTensor("F16", w.to(torch.float16).to(dev).contiguous(), (out_f, in_f))
    x = w.detach().float().cpu().numpy()
    if qtype == "FP8B":
        codes, scales = qref.quantize_fp8_block(x.reshape(-1), 128)
        return QTensor("FP8B", torch.from_numpy(codes.reshape(out_f, in_f)).to(dev), (out_f, in_f),
                       torch.from_numpy(scales.reshape(out_f, in_f // 128)).to(dev), 128)
    t = ggml_type(qtype)
    raw = qref.quantize(qtype, x.reshape(-1)).reshape(out_f, in_f // t.block_size * t.type_size)
    return QTensor(t.name, torch.from_numpy(raw.copy()).to(dev), (out_f, in_f))


@dataclass
class LinearWeight:
    """One logical projection made of row segments whose outputs are concatenated
    (e.g. fused q|k|v where v may use a different quant type in a Q4_K_M file)."""

    parts: List[QTensor]
    bias: Optional[torch.Tensor] = None
    # gate|up projection whose rows were interleaved per 128-row tile for the GEMM's SwiGLU epilogue
    swiglu_interleaved: bool = False

    @property
    def out_features(self) -> int:
        return sum(p.out_features for p in self.parts)

    @property
    def in_features(self) -> int:
        return self.parts[0].in_features

    def nbytes(self) -> int:
        return sum(p.nbytes() for p in self.parts)


# weight encodings the sm_100a kernels read directly (ops/cuda.py::QTYPE_CODE + the fp8-block path)
DEVICE_PACKED_TYPES = ("F32", "F16", "BF16", "Q8_0", "Q4_0", "Q4_K", "Q5_K", "Q6_K", "NVFP4", "FP8B")


def fuse_rows(parts: Sequence[QTensor]) -> List[QTensor]:
    """Concatenate adjacent segments that share an encoding into one tensor."""
    out: List[QTensor] = []
    for p in parts:
        if out and out[-1].qtype == p.qtype and out[-1].in_features == p.in_features and p.qtype != "FP8B":
            a = out[-1]
            out[-1] = QTensor(a.qtype, torch.cat([a.data, p.data], 0).contiguous(),
                              (a.out_features + p.out_features, a.in_features))
        else:
            out.append(p)
    return out


@dataclass
class ExpertWeights:
    """Stacked expert matrices ``[n_local_experts, rows, cols]`` (packed rows for quants)."""

    gate_up: List[QTensor]  # per local expert: fused [2*ffn, hidden]
    down: List[QTensor]
    first_expert: int = 0  # global id of local expert 0 (expert parallelism)
    gate_up_stack: Optional[QTensor] = None  # [(E*2ffn), hidden] rows of all local experts, expert-major
    down_stack: Optional[QTensor] = None

    def stack(self) -> bool:
        """Lay all local experts' rows out in one matrix per projection (what the grouped GEMM
        reads); the per-expert tensors become views of it, so nothing is held twice.  Returns False
        when the experts do not share one encoding."""
        if self.gate_up_stack is not None:
            return True
        for lst in (self.gate_up, self.down):
            if len({(q.qtype, q.shape) for q in lst}) != 1 or lst[0].qtype in ("FP8B", "F32", "F16"):
                return False
        for name in ("gate_up", "down"):
            lst = getattr(self, name)
            n, k = lst[0].shape
            data = torch.cat([q.data for q in lst], dim=0).contiguous()
            setattr(self, name + "_stack", QTensor(lst[0].qtype, data, (n * len(lst), k)))
            for i, q in enumerate(lst):
                q.data = data[i * n : (i + 1) * n]
        return True


@dataclass
class MLAWeights:
    """Latent-attention projections of one layer (this rank's heads).  The up-projection of the shared latent is kept
    per head and dense, split into its key part ``w_uk`` and value part ``w_uv``: the forward pass multiplies the queries
    by ``w_uk`` and the attention output by ``w_uv`` instead of rebuilding per-head keys and values."""

    kv_a: QTensor  # [kv_lora + rope, hidden]: latent and the shared rotary key
    kv_a_norm: torch.Tensor
    w_uk: torch.Tensor  # [heads, nope, kv_lora]
    w_uv: torch.Tensor  # [heads, v, kv_lora]
    q: Optional[LinearWeight] = None  # full query projection, or
    q_a: Optional[QTensor] = None  # down-projection,
    q_a_norm: Optional[torch.Tensor] = None
    q_b: Optional[LinearWeight] = None  # up-projection [heads * (nope + rope), q_lora]


@dataclass
class SSMWeights:
    """Mamba mixer: in_proj [2 d_inner, hidden] (rows: x then gate), depthwise kernel [d_inner, d_conv] + bias, x_proj
    [dt_rank + 2 d_state, d_inner], dt_proj [d_inner, dt_rank] + bias, A [d_inner, d_state] (already -exp(A_log)), D, out_proj."""

    in_proj: QTensor
    conv_kernel: torch.Tensor
    conv_bias: Optional[torch.Tensor]
    x_proj: QTensor
    dt_proj: QTensor
    dt_bias: torch.Tensor
    a: torch.Tensor
    d: torch.Tensor
    out_proj: LinearWeight


@dataclass
class GDNWeights:
    """Gated-delta-rule mixer (Qwen3.5): in_qkv [2 key_dim + value_dim, hidden], in_z [value_dim, hidden] (output gate),
    in_a / in_b [v_heads, hidden] (decay and write-strength inputs), depthwise kernel [2 key_dim + value_dim, taps],
    dt_bias and A (already -exp(A_log)) per value head, the gated norm's weight [head_v_dim], out_proj."""

    in_qkv: QTensor
    in_z: QTensor
    in_a: QTensor
    in_b: QTensor
    conv_kernel: torch.Tensor
    dt_bias: torch.Tensor
    a: torch.Tensor
    norm: torch.Tensor
    out_proj: LinearWeight


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    wqkv: Optional[LinearWeight]  # None in a latent-attention layer (``mla`` holds its projections) or a convolution layer
    wo: Optional[LinearWeight]
    ffn_norm: Optional[torch.Tensor]
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    mla: Optional[MLAWeights] = None
    # short-convolution mixer (LFM2) instead of attention: in_proj [3 hidden, hidden] (rows: B, C, x), depthwise kernel
    # [hidden, l_cache] (oldest tap first), out_proj [hidden, hidden]
    conv_in: Optional[QTensor] = None
    conv_kernel: Optional[torch.Tensor] = None
    conv_out: Optional[LinearWeight] = None
    gdn: Optional[GDNWeights] = None  # a gated-delta-rule layer in place of attention (the feed-forward block stays)
    ssm: Optional[SSMWeights] = None  # a state-space layer: no attention and no feed-forward block
    # Gemma-2/3: norms applied to the attention / FFN branch outputs before the residual add
    post_attn_norm: Optional[torch.Tensor] = None
    post_ffn_norm: Optional[torch.Tensor] = None
    # dense FFN
    w_gate_up: Optional[LinearWeight] = None
    w_down: Optional[LinearWeight] = None
    # MoE
    router: Optional[QTensor] = None
    router_bias: Optional[torch.Tensor] = None
    experts: Optional[ExpertWeights] = None
    shared_gate_up: Optional[LinearWeight] = None
    shared_down: Optional[LinearWeight] = None
    shared_gate: Optional[QTensor] = None
    norms_folded: bool = False  # attn_norm / ffn_norm were multiplied into wqkv / w_gate_up (Transformer._fold_norm_weights)


class StreamedLayers:
    """The decoder layers of a checkpoint held as a list that loads a layer from the file mapping when it is indexed
    and keeps at most ``capacity`` of them resident (least recently used goes first): a model whose layers do not fit
    next to the KV cache still runs, at the price of re-reading layers every step (the reference's layer-wise model,
    ``oxidize-core/src/model/layer_wise.rs``, with its LRU layer cache)."""

    def __init__(self, load, n_layers: int, capacity: int):
        from collections import OrderedDict

        if capacity < 1:
            raise ValueError("at least one layer has to be resident")
        self._load, self._n, self.capacity = load, n_layers, capacity
        self._cache: "OrderedDict[int, LayerWeights]" = OrderedDict()
        self.loads = 0
        self.evictions = 0

    def __len__(self) -> int:
        return self._n

    def __getitem__(self, i: int) -> "LayerWeights":
        if isinstance(i, slice):
            raise TypeError("streamed layers are indexed one at a time")
        if i < 0:
            i += self._n
        if not 0 <= i < self._n:
            raise IndexError(i)
        lw = self._cache.get(i)
        if lw is not None:
            self._cache.move_to_end(i)
            return lw
        while len(self._cache) >= self.capacity:
            self._cache.popitem(last=False)
            self.evictions += 1
        lw = self._load(i)
        self._cache[i] = lw
        self.loads += 1
        return lw

    def __iter__(self):
        return (self[i] for i in range(self._n))

    def resident(self) -> List["LayerWeights"]:
        return list(self._cache.values())


@dataclass
class MtpWeights:
    """``blk.L.nextn.*`` tensors of an in-GGUF multi-token-prediction head
    (``MtpWeights`` model/inference.rs:1403-1429)."""

    enorm: torch.Tensor
    hnorm: torch.Tensor
    eh_proj: QTensor
    layer: LayerWeights
    shared_head_norm: torch.Tensor
    shared_head: Optional[QTensor] = None
    embed: Optional[QTensor] = None


@dataclass
class ModelWeights:
    cfg: ModelConfig
    embed: QTensor
    layers: List[LayerWeights]
    out_norm: torch.Tensor
    lm_head: LinearWeight
    mtp: List[MtpWeights] = field(default_factory=list)
    tp_rank: int = 0
    tp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    first_layer: int = 0  # pipeline stage range [first_layer, first_layer+len(layers))
    vocab_start: int = 0  # first vocabulary row held by this rank's lm_head shard
    # per-pair divisors of the rotary frequencies stored in the checkpoint (Llama-3.1 ``rope_freqs.weight``,
    # Phi-3 LongRoPE ``rope_factors_short / _long.weight``), or None
    rope_freq_factors: Optional[torch.Tensor] = None
    rope_freq_factors_long: Optional[torch.Tensor] = None  # LongRoPE: used instead once the context exceeds the original one

    def nbytes(self) -> int:
        n = self.embed.nbytes() + self.lm_head.nbytes()
        for l in (self.layers.resident() if isinstance(self.layers, StreamedLayers) else self.layers):
            for lw in (l.wqkv, l.wo, l.w_gate_up, l.w_down, l.shared_gate_up, l.shared_down):
                if lw is not None:
                    n += lw.nbytes()
            if l.experts is not None:
                n += sum(e.nbytes() for e in l.experts.gate_up) + sum(e.nbytes() for e in l.experts.down)
        return n


# --------------------------------------------------------------------------- sharding helpers


def shard_range(n: int, rank: int, size: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous [start, stop) of ``n`` items for ``rank``; ``n`` must split into ``size``
    equal parts that are multiples of ``multiple``."""
    if n % (size * multiple):
        raise ValueError(f"cannot shard {n} into {size} parts of a multiple of {multiple}")
    per = n // size
    return rank * per, (rank + 1) * per


def _np_to_torch(a: np.ndarray, device, dtype=None) -> torch.Tensor:
    import warnings

    with warnings.catch_warnings():
        # read-only views of the GGUF mapping are never written through
        warnings.simplefilter("ignore", UserWarning)
        t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(device)


class GGUFWeightSource:
    """Reads (slices of) tensors from a GGUF mapping into device QTensors."""

    def __init__(self, g: GGUFFile, device, act_dtype: torch.dtype, transcode: str = ""):
        self.g = g
        # "Q8_0" / "Q4_0": weight matrices stored as floats are re-encoded in that block format on the way in
        self.transcode = transcode.upper()
        self.device = torch.device(device)
        self.act_dtype = act_dtype

    def has(self, name: str) -> bool:
        return self.g.has_tensor(name)

    def vector(self, name: str) -> torch.Tensor:
        info = self.g.tensors[name]
        x = qref.dequantize(info.type.name, self.g.tensor_bytes(name), info.n_elements)
        return torch.from_numpy(x.copy()).to(self.device, torch.float32)

    def matrix(self, name: str, rows: Optional[Tuple[int, int]] = None, cols: Optional[Tuple[int, int]] = None,
               expert: Optional[int] = None) -> QTensor:
        info = self.g.tensors[name]
        t: GGMLTypeInfo = info.type
        shape = info.shape
        in_f = shape[-1]
        out_f = shape[-2] if len(shape) >= 2 else 1
        raw = self.g.tensor_rows(name)  # [n_rows_total, row_nbytes]
        if len(shape) == 3:
            if expert is None:
                raise ValueError(f"{name} is a stacked expert tensor; pass expert=")
            raw = raw[expert * out_f : (expert + 1) * out_f]
        r0, r1 = rows if rows is not None else (0, out_f)
        raw = raw[r0:r1]
        c0, c1 = cols if cols is not None else (0, in_f)
        if (c0, c1) != (0, in_f):
            if c0 % t.block_size or c1 % t.block_size:
                raise ValueError(f"{name}: column shard [{c0},{c1}) not on {t.name} block boundary {t.block_size}")
            raw = raw[:, c0 // t.block_size * t.type_size : c1 // t.block_size * t.type_size]
        new_shape = (r1 - r0, c1 - c0)
        if (self.transcode and t.name in ("F32", "F16", "BF16") and new_shape[1] % 32 == 0 and new_shape[0] > 1
                and "token_embd" not in name and "ffn_gate_inp" not in name):
            x = qref.dequantize(t.name, np.ascontiguousarray(raw).reshape(-1), new_shape[0] * new_shape[1])
            tt = ggml_type(self.transcode)
            packed = qref.quantize(self.transcode, np.asarray(x, dtype=np.float32).reshape(-1))
            packed = np.ascontiguousarray(packed).view(np.uint8).reshape(new_shape[0], new_shape[1] // tt.block_size * tt.type_size)
            return QTensor(tt.name, _np_to_torch(packed, self.device), new_shape)
        if t.name == "F32":
            x = np.ascontiguousarray(raw).view("<f4")
            dt = torch.float32 if self.act_dtype == torch.float32 else torch.bfloat16
            return QTensor("F32" if dt == torch.float32 else "BF16", _np_to_torch(x, self.device, dt), new_shape)
        if t.name == "F16":
            x = np.ascontiguousarray(raw).view("<f2")
            if self.act_dtype == torch.float32:
                return QTensor("F32", _np_to_torch(x, self.device, torch.float32), new_shape)
            return QTensor("BF16", _np_to_torch(x, self.device, torch.bfloat16), new_shape)
        if t.name == "BF16":
            x = np.ascontiguousarray(raw).view("<i2")
            tt = torch.from_numpy(x).view(torch.bfloat16)
            if self.act_dtype == torch.float32:
                return QTensor("F32", tt.float().to(self.device), new_shape)
            return QTensor("BF16", tt.to(self.device), new_shape)
        if self.device.type == "cuda" and t.name not in DEVICE_PACKED_TYPES:
            # encodings the device kernels do not decode (Q2_K, Q3_K, Q4_1, Q5_0/1, IQ*) become bf16 at load time
            x = qref.dequantize(t.name, np.ascontiguousarray(raw).reshape(-1), new_shape[0] * new_shape[1])
            return QTensor("BF16", _np_to_torch(x.reshape(new_shape), self.device, torch.bfloat16), new_shape)
        return QTensor(t.name, _np_to_torch(raw, self.device), new_shape)


def _load_mla(src: GGUFWeightSource, cfg: ModelConfig, p: str, h0: int, h1: int) -> MLAWeights:
    """Latent-attention tensors of heads [h0, h1): ``attn_kv_b`` (rows = per head nope key rows, then value rows) or its
    split form ``attn_k_b`` ([head, kv_lora, nope], i.e. stored transposed) + ``attn_v_b`` ([head, v, kv_lora])."""
    from ..ops import ref as opref

    nope, vd, c, qk = cfg.qk_nope_dim, cfg.v_head_dim, cfg.kv_lora_rank, cfg.head_dim
    dt = src.act_dtype
    if src.has(f"{p}.attn_kv_b.weight"):
        kvb = opref.dequantize_weight(src.matrix(f"{p}.attn_kv_b.weight", rows=(h0 * (nope + vd), h1 * (nope + vd))))
        kvb = kvb.reshape(h1 - h0, nope + vd, c)
        w_uk, w_uv = kvb[:, :nope, :], kvb[:, nope:, :]
    else:
        w_uk = torch.stack([opref.dequantize_weight(src.matrix(f"{p}.attn_k_b.weight", expert=h)).t() for h in range(h0, h1)])
        w_uv = torch.stack([opref.dequantize_weight(src.matrix(f"{p}.attn_v_b.weight", expert=h)) for h in range(h0, h1)])
    m = MLAWeights(kv_a=src.matrix(f"{p}.attn_kv_a_mqa.weight"), kv_a_norm=src.vector(f"{p}.attn_kv_a_norm.weight"),
                   w_uk=w_uk.to(dt).contiguous(), w_uv=w_uv.to(dt).contiguous())
    if src.has(f"{p}.attn_q_a.weight"):
        m.q_a = src.matrix(f"{p}.attn_q_a.weight")
        m.q_a_norm = src.vector(f"{p}.attn_q_a_norm.weight")
        m.q_b = LinearWeight([src.matrix(f"{p}.attn_q_b.weight", rows=(h0 * qk, h1 * qk))])
    else:
        m.q = LinearWeight([src.matrix(f"{p}.attn_q.weight", rows=(h0 * qk, h1 * qk))])
    return m


def _load_ffn(src: "GGUFWeightSource", cfg: ModelConfig, p: str, lw: "LayerWeights", tp_rank: int, tp_size: int,
              ep_rank: int, ep_size: int) -> None:
    """The feed-forward half of layer ``p``: router + this rank's experts (+ shared expert), or one gated MLP."""
    if src.has(f"{p}.ffn_gate_inp.weight"):
        lw.router = src.matrix(f"{p}.ffn_gate_inp.weight")
        if src.has(f"{p}.exp_probs_b.bias"):
            lw.router_bias = src.vector(f"{p}.exp_probs_b.bias")
        e0, e1 = shard_range(cfg.n_experts, ep_rank, ep_size)
        gu, dn = [], []
        for e in range(e0, e1):
            g_ = src.matrix(f"{p}.ffn_gate_exps.weight", expert=e)
            u_ = src.matrix(f"{p}.ffn_up_exps.weight", expert=e)
            fused = fuse_rows([g_, u_])
            if len(fused) != 1:
                raise ValueError(f"{p}: expert gate/up use different encodings")
            gu.append(fused[0])
            dn.append(src.matrix(f"{p}.ffn_down_exps.weight", expert=e))
        lw.experts = ExpertWeights(gu, dn, e0)
        if src.has(f"{p}.ffn_gate_shexp.weight"):
            sf = cfg.shared_expert_ffn_size
            f0, f1 = shard_range(sf, tp_rank, tp_size, 256 if sf % (256 * tp_size) == 0 else 1)
            lw.shared_gate_up = LinearWeight(fuse_rows([src.matrix(f"{p}.ffn_gate_shexp.weight", rows=(f0, f1)),
                                                        src.matrix(f"{p}.ffn_up_shexp.weight", rows=(f0, f1))]))
            lw.shared_down = LinearWeight([src.matrix(f"{p}.ffn_down_shexp.weight", cols=(f0, f1))])
            if src.has(f"{p}.ffn_gate_inp_shexp.weight"):
                lw.shared_gate = src.matrix(f"{p}.ffn_gate_inp_shexp.weight")
    elif not src.has(f"{p}.ffn_gate.weight"):
        # fused gate / up tensor (Phi-3): the first half of the rows is the gate, the second half the up projection
        ffn = src.g.tensors[f"{p}.ffn_up.weight"].shape[0] // 2
        f0, f1 = shard_range(ffn, tp_rank, tp_size)
        lw.w_gate_up = LinearWeight(fuse_rows([src.matrix(f"{p}.ffn_up.weight", rows=(f0, f1)),
                                               src.matrix(f"{p}.ffn_up.weight", rows=(ffn + f0, ffn + f1))]))
        lw.w_down = LinearWeight([src.matrix(f"{p}.ffn_down.weight", cols=(f0, f1))])
    else:
        ffn = src.g.tensors[f"{p}.ffn_gate.weight"].shape[0]
        f0, f1 = shard_range(ffn, tp_rank, tp_size)
        lw.w_gate_up = LinearWeight(fuse_rows([src.matrix(f"{p}.ffn_gate.weight", rows=(f0, f1)),
                                               src.matrix(f"{p}.ffn_up.weight", rows=(f0, f1))]))
        lw.w_down = LinearWeight([src.matrix(f"{p}.ffn_down.weight", cols=(f0, f1))])


def _load_layer(src: GGUFWeightSource, cfg: ModelConfig, i: int, tp_rank: int, tp_size: int,
                ep_rank: int, ep_size: int, prefix: Optional[str] = None) -> LayerWeights:
    p = prefix or f"blk.{i}"
    hd = cfg.head_dim
    # attention heads are sharded by KV head; with fewer KV heads than ranks they replicate
    kv_rep = max(1, tp_size // cfg.n_kv_heads)
    kv_shards = min(tp_size, cfg.n_kv_heads)
    q0, q1 = shard_range(cfg.n_heads, tp_rank, tp_size)
    k0, k1 = shard_range(cfg.n_kv_heads, tp_rank // kv_rep, kv_shards)
    qr, kr = (q0 * hd, q1 * hd), (k0 * hd, k1 * hd)
    mla = None
    if src.has(f"{p}.ssm_in.weight"):
        if tp_size > 1:
            raise ValueError("state-space layers are not sharded: run this model with tp_size = 1")
        di = cfg.ssm_d_inner
        ssm = SSMWeights(in_proj=src.matrix(f"{p}.ssm_in.weight"), conv_kernel=src.vector(f"{p}.ssm_conv1d.weight").reshape(di, -1),
                         conv_bias=src.vector(f"{p}.ssm_conv1d.bias") if src.has(f"{p}.ssm_conv1d.bias") else None,
                         x_proj=src.matrix(f"{p}.ssm_x.weight"), dt_proj=src.matrix(f"{p}.ssm_dt.weight"),
                         dt_bias=src.vector(f"{p}.ssm_dt.bias"), a=src.vector(f"{p}.ssm_a").reshape(di, -1),
                         d=src.vector(f"{p}.ssm_d"), out_proj=LinearWeight([src.matrix(f"{p}.ssm_out.weight")]))
        return LayerWeights(attn_norm=src.vector(f"{p}.attn_norm.weight"), wqkv=None, wo=None, ffn_norm=None, ssm=ssm)
    # the norm in front of the feed-forward block; Qwen3.5 files name it post_attention_norm
    ffn_norm_name = f"{p}.ffn_norm.weight" if src.has(f"{p}.ffn_norm.weight") or not cfg.attn_out_gate else f"{p}.post_attention_norm.weight"
    if src.has(f"{p}.ssm_alpha.weight"):
        if tp_size > 1:
            raise ValueError("gated-delta-rule layers are not sharded: run this model with tp_size = 1")
        rows = src.g.tensors[f"{p}.attn_qkv.weight"].shape[0]
        gdn = GDNWeights(in_qkv=src.matrix(f"{p}.attn_qkv.weight"), in_z=src.matrix(f"{p}.attn_gate.weight"),
                         in_a=src.matrix(f"{p}.ssm_alpha.weight"), in_b=src.matrix(f"{p}.ssm_beta.weight"),
                         conv_kernel=src.vector(f"{p}.ssm_conv1d.weight").reshape(rows, -1),
                         dt_bias=src.vector(f"{p}.ssm_dt.bias"), a=src.vector(f"{p}.ssm_a").reshape(-1),
                         norm=src.vector(f"{p}.ssm_norm.weight"), out_proj=LinearWeight([src.matrix(f"{p}.ssm_out.weight")]))
        lw = LayerWeights(attn_norm=src.vector(f"{p}.attn_norm.weight"), wqkv=None, wo=None, ffn_norm=src.vector(ffn_norm_name), gdn=gdn)
        _load_ffn(src, cfg, p, lw, tp_rank, tp_size, ep_rank, ep_size)
        return lw
    if src.has(f"{p}.shortconv.conv.weight"):
        if tp_size > 1:
            raise ValueError("short-convolution layers are not sharded: run this model with tp_size = 1")
        lw = LayerWeights(attn_norm=src.vector(f"{p}.attn_norm.weight"), wqkv=None, wo=None,
                          ffn_norm=src.vector(f"{p}.ffn_norm.weight"), conv_in=src.matrix(f"{p}.shortconv.in_proj.weight"),
                          conv_kernel=src.vector(f"{p}.shortconv.conv.weight").reshape(cfg.hidden_size, -1),
                          conv_out=LinearWeight([src.matrix(f"{p}.shortconv.out_proj.weight")]))
        _load_ffn(src, cfg, p, lw, tp_rank, tp_size, ep_rank, ep_size)  # dense, or routed experts (LFM2-MoE)
        return lw
    if src.has(f"{p}.attn_kv_a_mqa.weight"):
        mla = _load_mla(src, cfg, p, q0, q1)
        parts = []
    elif src.has(f"{p}.attn_qkv.weight"):
        # one fused tensor (Phi-3): rows are all query heads, then all key heads, then all value heads
        ko, vo = cfg.n_heads * hd, (cfg.n_heads + cfg.n_kv_heads) * hd
        parts = [src.matrix(f"{p}.attn_qkv.weight", rows=qr), src.matrix(f"{p}.attn_qkv.weight", rows=(ko + kr[0], ko + kr[1])),
                 src.matrix(f"{p}.attn_qkv.weight", rows=(vo + kr[0], vo + kr[1]))]
    elif cfg.attn_out_gate:
        if tp_size > 1:
            raise ValueError("gated attention is not sharded: run this model with tp_size = 1")
        # per head: the query rows, then the rows of that head's output gate
        parts = [src.matrix(f"{p}.attn_q.weight"), src.matrix(f"{p}.attn_k.weight", rows=kr), src.matrix(f"{p}.attn_v.weight", rows=kr)]
    else:
        parts = [src.matrix(f"{p}.attn_q.weight", rows=qr), src.matrix(f"{p}.attn_k.weight", rows=kr),
                 src.matrix(f"{p}.attn_v.weight", rows=kr)]
    bias = None
    if src.has(f"{p}.attn_qkv.bias"):
        b = src.vector(f"{p}.attn_qkv.bias")
        ko, vo = cfg.n_heads * hd, (cfg.n_heads + cfg.n_kv_heads) * hd
        bias = torch.cat([b[qr[0]:qr[1]], b[ko + kr[0]:ko + kr[1]], b[vo + kr[0]:vo + kr[1]]])
    elif src.has(f"{p}.attn_q.bias"):
        bias = torch.cat([src.vector(f"{p}.attn_q.bias")[qr[0]:qr[1]], src.vector(f"{p}.attn_k.bias")[kr[0]:kr[1]],
                          src.vector(f"{p}.attn_v.bias")[kr[0]:kr[1]]])
    vd = cfg.v_head_dim if mla is not None else hd
    lw = LayerWeights(
        attn_norm=src.vector(f"{p}.attn_norm.weight"),
        wqkv=LinearWeight(fuse_rows(parts), bias) if mla is None else None,
        wo=LinearWeight([src.matrix(f"{p}.attn_output.weight", cols=(q0 * vd, q1 * vd))]),
        ffn_norm=src.vector(ffn_norm_name),
        mla=mla,
    )
    if src.has(f"{p}.attn_q_norm.weight"):
        lw.q_norm = src.vector(f"{p}.attn_q_norm.weight")
        lw.k_norm = src.vector(f"{p}.attn_k_norm.weight")
    if src.has(f"{p}.post_attention_norm.weight") and ffn_norm_name.endswith("ffn_norm.weight"):
        lw.post_attn_norm = src.vector(f"{p}.post_attention_norm.weight")
    if src.has(f"{p}.post_ffw_norm.weight"):
        lw.post_ffn_norm = src.vector(f"{p}.post_ffw_norm.weight")
    _load_ffn(src, cfg, p, lw, tp_rank, tp_size, ep_rank, ep_size)
    return lw


def load_weights(g: GGUFFile, cfg: ModelConfig, device="cpu", act_dtype: torch.dtype = torch.float32,
                 tp_rank: int = 0, tp_size: int = 1, ep_rank: int = 0, ep_size: int = 1,
                 layer_range: Optional[Tuple[int, int]] = None, resident_layers: int = 0, transcode: str = "") -> ModelWeights:
    """Load this rank's shard of a GGUF checkpoint.

    ``layer_range`` selects a pipeline stage (only its own tensors are read, unlike the
    reference's two-node pipeline where both nodes map the whole file, pipeline.rs:23).
    ``resident_layers`` > 0 keeps only that many decoder layers loaded at a time (:class:`StreamedLayers`)."""
    if transcode and transcode.upper() not in ("Q8_0", "Q4_0"):
        raise ValueError("weights can be re-encoded at load time as Q8_0 or Q4_0")
    src = GGUFWeightSource(g, device, act_dtype, transcode)
    l0, l1 = layer_range if layer_range is not None else (0, cfg.n_layers)
    if resident_layers > 0 and resident_layers < l1 - l0:
        layers = StreamedLayers(lambda i: _load_layer(src, cfg, l0 + i, tp_rank, tp_size, ep_rank, ep_size), l1 - l0,
                                resident_layers)
    else:
        layers = [_load_layer(src, cfg, i, tp_rank, tp_size, ep_rank, ep_size) for i in range(l0, l1)]
    embed = src.matrix("token_embd.weight")
    v0, v1 = shard_range(cfg.vocab_size, tp_rank, tp_size) if cfg.vocab_size % tp_size == 0 else (0, cfg.vocab_size)
    head_name = "output.weight" if src.has("output.weight") else "token_embd.weight"
    lm_head = LinearWeight([src.matrix(head_name, rows=(v0, v1))])
    norm_name = "output_norm.weight" if src.has("output_norm.weight") else "token_embd_norm.weight"  # LFM2 files use the latter
    mw = ModelWeights(cfg, embed, layers, src.vector(norm_name), lm_head, [], tp_rank, tp_size,
                      ep_rank, ep_size, l0, v0)
    if src.has("rope_freqs.weight"):
        mw.rope_freq_factors = src.vector("rope_freqs.weight")
    elif src.has("rope_factors_short.weight"):
        mw.rope_freq_factors = src.vector("rope_factors_short.weight")
        if src.has("rope_factors_long.weight"):
            mw.rope_freq_factors_long = src.vector("rope_factors_long.weight")
    for j in range(cfg.nextn_layers):
        L = cfg.n_layers + j
        p = f"blk.{L}.nextn"
        if not src.has(f"{p}.eh_proj.weight"):
            continue
        mw.mtp.append(MtpWeights(
            enorm=src.vector(f"{p}.enorm.weight"), hnorm=src.vector(f"{p}.hnorm.weight"),
            eh_proj=src.matrix(f"{p}.eh_proj.weight"),
            layer=_load_layer(src, cfg, L, tp_rank, tp_size, ep_rank, ep_size),
            shared_head_norm=src.vector(f"{p}.shared_head_norm.weight"),
            shared_head=src.matrix(f"{p}.shared_head_head.weight") if src.has(f"{p}.shared_head_head.weight") else None,
            embed=src.matrix(f"{p}.embed_tokens.weight") if src.has(f"{p}.embed_tokens.weight") else None))
    return mw
