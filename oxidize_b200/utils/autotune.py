"""Hardware detection → model fingerprint → tuning plan, as a pure function with a rationale log.

Same three-step shape as the reference autotuner (``oxidize-core/src/autotune/rules.rs:1-63``:
``detect()`` → ``fingerprint(gguf)`` → ``plan()``; "explicit beats implicit": the plan only
fills flags the user did not pass, ``main/inference.rs:51``), but the rules target one box of
B200s: how many GPUs to shard over, which KV encoding fits, how many KV pages to allocate, and
a bandwidth-roofline decode estimate instead of the reference's constant (200 tok/s for B200,
``rules.rs:517-533``).
"""
from __future__ import annotations

import json
import os
import subprocess
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional

from ..formats.gguf import GGUFFile
from ..models.config import ModelConfig, config_from_gguf

B200_HBM_GBS = 6555.0  # sustained copy bandwidth of a B200 (HBM3e), GB/s: the bound the decode estimates use


@dataclass
class GpuInfo:
    index: int
    name: str
    memory_bytes: int


@dataclass
class HardwareInventory:
    physical_cores: int = 1
    total_ram_bytes: int = 0
    gpus: List[GpuInfo] = field(default_factory=list)

    @property
    def has_gpu(self) -> bool:
        return bool(self.gpus)


def parse_nvidia_smi_csv(text: str) -> List[GpuInfo]:
    """Parse ``nvidia-smi --query-gpu=index,name,memory.total --format=csv,noheader,nounits``."""
    out = []
    for line in text.strip().splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) >= 3 and f[0].isdigit():
            try:
                out.append(GpuInfo(int(f[0]), f[1], int(float(f[2])) * (1 << 20)))
            except ValueError:
                continue
    return out


def detect(run=subprocess.run) -> HardwareInventory:
    inv = HardwareInventory(physical_cores=os.cpu_count() or 1)
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemTotal:"):
                    inv.total_ram_bytes = int(line.split()[1]) * 1024
                    break
    except OSError:
        pass
    try:
        r = run(["nvidia-smi", "--query-gpu=index,name,memory.total", "--format=csv,noheader,nounits"],
                capture_output=True, text=True, timeout=10)
        if r.returncode == 0:
            inv.gpus = parse_nvidia_smi_csv(r.stdout)
    except (OSError, subprocess.SubprocessError):
        pass
    return inv


@dataclass
class ModelFingerprint:
    arch: str
    n_layers: int
    hidden_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    is_moe: bool
    n_experts: int
    weight_bytes: int
    context_length: int
    has_mtp: bool
    dominant_quant: str


def fingerprint(g: GGUFFile, cfg: Optional[ModelConfig] = None) -> ModelFingerprint:
    cfg = cfg or config_from_gguf(g)
    by_type: Dict[str, int] = {}
    total = 0
    for info in g.tensors.values():
        by_type[info.type.name] = by_type.get(info.type.name, 0) + info.nbytes
        total += info.nbytes
    dom = max(by_type, key=by_type.get) if by_type else "F32"
    # what one token's cache row holds: KV heads x head_dim, or with latent attention one shared (latent + rotary key) row
    kv_heads, kv_dim = (1, cfg.kv_lora_rank + cfg.rotary_dim) if cfg.is_mla else (cfg.n_kv_heads, cfg.head_dim)
    return ModelFingerprint(cfg.arch, cfg.n_layers, cfg.hidden_size, cfg.n_heads, kv_heads, kv_dim,
                            cfg.is_moe, cfg.n_experts, total, cfg.context_length, cfg.nextn_layers > 0, dom)


@dataclass
class TuningPlan:
    backend: str = "cpu"
    tp_size: int = 1
    kv_cache_dtype: str = "f32"
    ctx_size: int = 4096
    max_num_seqs: int = 8
    num_kv_blocks: int = 0
    prefill_chunk_size: int = 512
    cuda_graphs: bool = True
    speculative: str = "none"  # none | mtp | draft
    threads: int = 0
    expected_decode_tps: float = 0.0
    expected_prompt_tps: float = 0.0
    rationale: List[str] = field(default_factory=list)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2)

    def render(self) -> str:
        lines = [f"backend={self.backend} tp={self.tp_size} kv={self.kv_cache_dtype} ctx={self.ctx_size} "
                 f"max_seqs={self.max_num_seqs} kv_blocks={self.num_kv_blocks} spec={self.speculative}",
                 f"expected: prompt {self.expected_prompt_tps:.0f} tok/s, decode {self.expected_decode_tps:.0f} tok/s"]
        if self.rationale:
            lines.append("Rationale:")
            lines += [f"  - {r}" for r in self.rationale]
        return "\n".join(lines)


def kv_bytes_per_token(m: ModelFingerprint, kv_dtype: str, tp: int) -> int:
    heads = max(1, m.n_kv_heads // tp)
    per = {"f32": 4.0, "f16": 2.0, "bf16": 2.0, "q8": 1.0 + 4 / 32, "q4": 0.5 + 4 / 32}[kv_dtype]
    return int(m.n_layers * heads * 2 * m.head_dim * per)


def plan(inv: HardwareInventory, m: ModelFingerprint, want_ctx: int = 0, want_seqs: int = 0) -> TuningPlan:
    p = TuningPlan()
    r = p.rationale
    ctx = want_ctx or min(m.context_length or 4096, 8192)
    p.ctx_size = ctx
    if not inv.has_gpu:
        p.backend, p.kv_cache_dtype, p.cuda_graphs = "cpu", "f16", False
        p.threads = inv.physical_cores
        p.max_num_seqs = want_seqs or 4
        r.append("no GPU found → CPU reference path, f16 KV")
        mem_tps = (inv.total_ram_bytes * 0.0 + 20e9) / max(m.weight_bytes, 1)
        p.expected_decode_tps = mem_tps
        p.expected_prompt_tps = mem_tps * 6
        return p
    p.backend = "cuda"
    gpu_mem = min(g.memory_bytes for g in inv.gpus)
    usable = int(gpu_mem * 0.90)
    n = len(inv.gpus)
    # tier: how many GPUs — smallest power of two whose shards leave >= 25 % of memory for KV
    tp = 1
    while tp < n and m.weight_bytes / tp > usable * 0.75:
        tp *= 2
    while tp > 1 and (m.n_heads % tp or (m.n_kv_heads % tp and tp % m.n_kv_heads)):
        tp //= 2
    p.tp_size = tp
    r.append(f"{m.weight_bytes / 1e9:.1f} GB of weights over {tp} GPU(s) of {gpu_mem / 1e9:.0f} GB")
    # tier: KV encoding
    seqs = want_seqs or 64
    free = usable - m.weight_bytes / tp
    for kvd in ("bf16", "q8", "q4"):
        need = kv_bytes_per_token(m, kvd, tp) * ctx * seqs
        if need <= free:
            p.kv_cache_dtype = kvd
            break
    else:
        p.kv_cache_dtype = "q4"
        seqs = max(1, int(free // max(kv_bytes_per_token(m, "q4", tp) * ctx, 1)))
        r.append(f"KV does not fit {want_seqs or 64} sequences even at q4 → {seqs} sequences")
    if p.kv_cache_dtype != "bf16":
        r.append(f"bf16 KV for {seqs}×{ctx} tokens exceeds the {free / 1e9:.0f} GB left → {p.kv_cache_dtype} KV")
    p.max_num_seqs = seqs
    p.num_kv_blocks = int(min(free // max(kv_bytes_per_token(m, p.kv_cache_dtype, tp) * 16, 1),
                              seqs * (ctx // 16 + 1)))
    p.speculative = "mtp" if m.has_mtp else "none"
    if m.has_mtp:
        r.append("model ships nextn layers → MTP speculative decoding")
    # bandwidth roofline for batch-1 decode; prefill is compute-bound, coarse 6× as in the reference
    p.expected_decode_tps = B200_HBM_GBS * 1e9 * tp / max(m.weight_bytes, 1) * 0.6
    p.expected_prompt_tps = p.expected_decode_tps * 6
    r.append("decode estimate = 60 % of (HBM bandwidth × GPUs ÷ weight bytes)")
    return p


def apply_plan(args: Dict[str, Any], user_set: set, p: TuningPlan) -> Dict[str, Any]:
    """Fill only what the user did not pass ("explicit beats implicit")."""
    mapping = {"backend": p.backend, "tp": p.tp_size, "kv_cache_dtype": p.kv_cache_dtype, "ctx_size": p.ctx_size,
               "max_running": p.max_num_seqs, "threads": p.threads}
    out = dict(args)
    for k, v in mapping.items():
        if k not in user_set:
            out[k] = v
    return out


# --------------------------------------------------------------------------- prefill token budget


def plan_resident_layers(n_layers: int, layer_bytes: int, fixed_bytes: int, kv_bytes: int, budget_bytes: int) -> int:
    """How many decoder layers to keep loaded when the whole model may not fit beside its cache (``--ram-offload``; the
    reference's offload planner, ``model/offload.rs:66-95``): 0 = everything fits, otherwise the largest count that leaves
    room for the embedding / head (``fixed_bytes``), the KV cache and one layer in flight; at least one."""
    if n_layers * layer_bytes + fixed_bytes + kv_bytes <= budget_bytes:
        return 0
    room = budget_bytes - fixed_bytes - kv_bytes - layer_bytes  # one more layer's worth while the next one loads
    return max(1, min(n_layers - 1, room // max(layer_bytes, 1)))


def prefill_token_budget(cfg: ModelConfig, tp: int = 1, sm_count: int = 148, lo: int = 2048, hi: int = 3072,
                         token_tile: int = 256, row_tile: int = 128) -> int:
    """Tokens per engine step (prefill chunks + decode rows) that waste the fewest tensor-core tiles.

    A prefill-sized projection runs ``ceil(N / 128) x ceil(T / 256)`` tiles, one per SM at a time, so its cost is a
    whole number of waves of ``sm_count`` tiles and the last wave is paid in full however empty it is.  For every
    multiple of the token tile in [lo, hi] the useful work of the four projections of a layer (per-rank shapes under
    ``tp``-way tensor parallelism) is divided by the work of the waves they occupy; the budget with the best ratio
    wins, the smaller one on ties (shorter steps delay the running sequences' decode rows less).  Measured on the
    per-rank shapes of the 70B model under TP8, one B200: 2304 tokens prefill 5 % faster than 2048, 3072 tokens 7 %,
    4096 tokens 8 % slower (larger attention tiles); hence the default upper bound.

    The reference has no counterpart: its engines prefill one sequence at a time in fixed tiles
    (``oxidize-c/src/compute/matvec.c:934-937`` tunes the activation-tile size instead)."""
    tp = max(1, int(tp))
    h, hd = cfg.hidden_size, cfg.head_dim
    ffn = cfg.expert_ffn_size * max(cfg.n_experts_used, 1) if cfg.is_moe and cfg.expert_ffn_size else cfg.ffn_size
    shapes = [  # (output rows per rank, input columns per rank)
        ((cfg.n_heads + 2 * cfg.n_kv_heads) * hd // tp, h),
        (h, cfg.n_heads * hd // tp),
        (2 * ffn // tp, h),
        (h, max(ffn // tp, 1)),
    ]
    best, best_eff = lo, -1.0
    t = (lo + token_tile - 1) // token_tile * token_tile
    while t <= hi:
        useful = cost = 0.0
        for n, k in shapes:
            tiles = -(-n // row_tile) * -(-t // token_tile)
            waves = -(-tiles // sm_count)
            useful += float(n) * k * t
            cost += float(waves) * sm_count * row_tile * token_tile * k
        eff = useful / cost if cost else 0.0
        if eff > best_eff + 1e-9:
            best, best_eff = t, eff
        t += token_tile
    return best
