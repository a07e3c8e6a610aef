"""CLIP-style vision tower + multimodal projector.

The reference's encoder (``oxidize-core/src/vision/encoder.rs:67-125``) is the embedding stage alone: patch projection,
class token, position embeddings, one norm and a projection; its config (``vision/config.rs:10-21``) already names the
transformer's sizes (heads, layers, MLP width).  Here the whole tower runs: patch embedding, class token, learned
positions, pre-LayerNorm, ``num_hidden_layers`` pre-norm blocks (biased q/k/v/out attention over all patches, quick-GELU
or GELU MLP), and the LLaVA read-out: the hidden states after a chosen block (second to last by default), class token
dropped, through a linear-GELU-linear projector whose output rows are the image's tokens in the language model's
embedding space.  Weights load from a llama.cpp-style projector file (``v.*`` / ``mm.*`` tensors, ``clip.vision.*`` keys);
``convert_vision_tower`` writes one from a Hugging Face LLaVA directory.  The math is plain torch on the model's device
(dense attention over a few hundred patches, once per image).
"""
from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..formats.gguf import GGUFValueType, GGUFWriter, load_gguf
from ..formats.safetensors_io import SafeTensorsFile

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class VisionConfig:
    image_size: int = 336
    patch_size: int = 14
    hidden_size: int = 1024
    num_attention_heads: int = 16
    num_hidden_layers: int = 24
    intermediate_size: int = 4096
    layer_norm_eps: float = 1e-5
    projection_dim: int = 4096  # the language model's hidden size
    image_mean: Tuple[float, float, float] = CLIP_MEAN
    image_std: Tuple[float, float, float] = CLIP_STD
    feature_layer: int = -2  # which block's output feeds the projector (negative: from the end)
    use_gelu: bool = False  # False: quick-GELU (x * sigmoid(1.702 x)), CLIP's activation

    @classmethod
    def clip_large(cls) -> "VisionConfig":
        return cls(image_size=224, projection_dim=768)

    @classmethod
    def clip_base(cls) -> "VisionConfig":
        return cls(image_size=224, patch_size=16, hidden_size=768, num_attention_heads=12, num_hidden_layers=12,
                   intermediate_size=3072, projection_dim=512)

    @classmethod
    def llava_1_5(cls) -> "VisionConfig":
        return cls()

    @property
    def num_patches_per_side(self) -> int:
        return self.image_size // self.patch_size

    @property
    def num_patches(self) -> int:
        return self.num_patches_per_side ** 2

    @property
    def num_image_tokens(self) -> int:
        return self.num_patches  # the class token is dropped

    @property
    def patch_dim(self) -> int:
        return 3 * self.patch_size * self.patch_size

    def validate(self) -> None:
        if self.image_size <= 0 or self.patch_size <= 0 or self.image_size % self.patch_size:
            raise ValueError("image_size must be a positive multiple of patch_size")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must divide into the attention heads")
        if not -self.num_hidden_layers - 1 <= self.feature_layer <= self.num_hidden_layers:
            raise ValueError("feature_layer outside the tower")


class ImagePreprocessor:
    """RGB(A) image → normalised ``[3, S, S]`` tensor: resize the shorter side to S (bicubic), centre crop, scale to [0, 1],
    subtract the mean and divide by the standard deviation per channel (the CLIP recipe; the reference's
    ``vision/preprocess.rs:36-62`` resizes with nearest-neighbour sampling)."""

    def __init__(self, config: VisionConfig):
        self.config = config

    def __call__(self, image) -> torch.Tensor:
        a = np.asarray(image)
        if a.ndim == 2:
            a = np.repeat(a[:, :, None], 3, axis=2)
        if a.ndim != 3 or a.shape[2] not in (3, 4):
            raise ValueError("image must be H x W x 3 (or 4) values")
        a = a[:, :, :3]
        x = torch.from_numpy(np.ascontiguousarray(a)).permute(2, 0, 1).float()
        if a.dtype == np.uint8:
            x = x / 255.0
        S = self.config.image_size
        _, h, w = x.shape
        if (h, w) != (S, S):
            s = S / min(h, w)
            nh, nw = max(S, round(h * s)), max(S, round(w * s))
            x = F.interpolate(x[None], size=(nh, nw), mode="bicubic", align_corners=False, antialias=True)[0].clamp(0, 1)
            top, left = (nh - S) // 2, (nw - S) // 2
            x = x[:, top : top + S, left : left + S]
        mean = torch.tensor(self.config.image_mean)[:, None, None]
        std = torch.tensor(self.config.image_std)[:, None, None]
        return (x - mean) / std

    def patches(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[3, S, S]`` → ``[num_patches, 3 * p * p]`` rows in raster order (channel-major inside a patch), the layout the
        patch projection multiplies."""
        p, g = self.config.patch_size, self.config.num_patches_per_side
        return pixels.reshape(3, g, p, g, p).permute(1, 3, 0, 2, 4).reshape(g * g, 3 * p * p)


@dataclass
class _Block:
    ln1: Tuple[torch.Tensor, torch.Tensor]
    ln2: Tuple[torch.Tensor, torch.Tensor]
    q: Tuple[torch.Tensor, torch.Tensor]
    k: Tuple[torch.Tensor, torch.Tensor]
    v: Tuple[torch.Tensor, torch.Tensor]
    o: Tuple[torch.Tensor, torch.Tensor]
    fc1: Tuple[torch.Tensor, torch.Tensor]
    fc2: Tuple[torch.Tensor, torch.Tensor]


@dataclass
class VisionEncoder:
    config: VisionConfig
    patch_embedding: torch.Tensor  # [hidden, 3 * p * p]
    class_token: torch.Tensor
    position_embeddings: torch.Tensor  # [num_patches + 1, hidden]
    pre_ln: Tuple[torch.Tensor, torch.Tensor]
    blocks: List[_Block] = field(default_factory=list)
    post_ln: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
    projector: List[Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=list)  # linear layers, GELU between them

    def hidden_states(self, pixels: torch.Tensor) -> List[torch.Tensor]:
        """``pixels`` [3, S, S] → the residual stream after the embedding stage and after every block, each
        [num_patches + 1, hidden] (index 0 = the class token)."""
        c = self.config
        pre = ImagePreprocessor(c)
        x = pre.patches(pixels.to(self.patch_embedding.device, torch.float32)) @ self.patch_embedding.t()
        x = torch.cat([self.class_token[None, :], x], dim=0) + self.position_embeddings
        x = F.layer_norm(x, (c.hidden_size,), self.pre_ln[0], self.pre_ln[1], c.layer_norm_eps)
        out = [x]
        nh = c.num_attention_heads
        hd = c.hidden_size // nh
        for b in self.blocks:
            h = F.layer_norm(x, (c.hidden_size,), b.ln1[0], b.ln1[1], c.layer_norm_eps)
            q = (h @ b.q[0].t() + b.q[1]).reshape(-1, nh, hd).transpose(0, 1)
            k = (h @ b.k[0].t() + b.k[1]).reshape(-1, nh, hd).transpose(0, 1)
            v = (h @ b.v[0].t() + b.v[1]).reshape(-1, nh, hd).transpose(0, 1)
            a = torch.softmax(q @ k.transpose(1, 2) * hd ** -0.5, dim=-1) @ v
            x = x + (a.transpose(0, 1).reshape(-1, c.hidden_size) @ b.o[0].t() + b.o[1])
            h = F.layer_norm(x, (c.hidden_size,), b.ln2[0], b.ln2[1], c.layer_norm_eps)
            h = h @ b.fc1[0].t() + b.fc1[1]
            h = F.gelu(h) if c.use_gelu else h * torch.sigmoid(1.702 * h)
            x = x + (h @ b.fc2[0].t() + b.fc2[1])
            out.append(x)
        return out

    def encode(self, pixels: torch.Tensor) -> torch.Tensor:
        """Image tokens for the language model: [num_patches, projection_dim] float32."""
        hs = self.hidden_states(pixels)
        x = hs[self.config.feature_layer][1:]  # the class token is dropped
        for i, (w, b) in enumerate(self.projector):
            if i:
                x = F.gelu(x)
            x = x @ w.t() + b
        return x


# --------------------------------------------------------------------------- files

_BLOCK_PARTS = {"ln1": "ln1", "ln2": "ln2", "q": "attn_q", "k": "attn_k", "v": "attn_v", "o": "attn_out", "fc1": "ffn_up",
                "fc2": "ffn_down"}


def load_vision_encoder(path: str, device="cpu") -> VisionEncoder:
    g = load_gguf(path)

    def md(key, default=None):
        return g.metadata.get(f"clip.vision.{key}", g.metadata.get(f"clip.{key}", default))

    cfg = VisionConfig(image_size=int(md("image_size")), patch_size=int(md("patch_size")), hidden_size=int(md("embedding_length")),
                       num_attention_heads=int(md("attention.head_count")), num_hidden_layers=int(md("block_count")),
                       intermediate_size=int(md("feed_forward_length")), layer_norm_eps=float(md("attention.layer_norm_epsilon", 1e-5)),
                       projection_dim=int(md("projection_dim")), image_mean=tuple(md("image_mean", CLIP_MEAN)),
                       image_std=tuple(md("image_std", CLIP_STD)), feature_layer=int(md("feature_layer", -2)),
                       use_gelu=bool(md("use_gelu", False)))
    cfg.validate()
    from ..quant import ref as qref

    def t(name) -> torch.Tensor:
        info = g.tensors[name]
        x = qref.dequantize(info.type.name, np.ascontiguousarray(g.tensor_bytes(name)), info.n_elements)
        return torch.from_numpy(np.asarray(x, dtype=np.float32).reshape(info.shape).copy()).to(device)

    def pair(prefix) -> Tuple[torch.Tensor, torch.Tensor]:
        w = t(prefix + ".weight")
        return w, (t(prefix + ".bias") if g.has_tensor(prefix + ".bias") else torch.zeros(w.shape[0], device=device))

    blocks = []
    for i in range(cfg.num_hidden_layers):
        if not g.has_tensor(f"v.blk.{i}.attn_q.weight"):
            break  # files may leave out the blocks after the feature layer
        parts = {k: pair(f"v.blk.{i}.{n}") for k, n in _BLOCK_PARTS.items()}
        if parts["fc1"][0].shape[0] != cfg.intermediate_size:  # older converters wrote the two MLP matrices under each other's name
            parts["fc1"], parts["fc2"] = parts["fc2"], parts["fc1"]
        blocks.append(_Block(**parts))
    proj = []
    for i in range(0, 8, 2):
        if g.has_tensor(f"mm.{i}.weight"):
            proj.append(pair(f"mm.{i}"))
    if proj and proj[-1][0].shape[0] != cfg.projection_dim:
        raise ValueError("projector output width does not match clip.vision.projection_dim")
    return VisionEncoder(cfg, t("v.patch_embd.weight").reshape(cfg.hidden_size, -1), t("v.class_embd"), t("v.position_embd.weight"),
                         pair("v.pre_ln"), blocks, pair("v.post_ln") if g.has_tensor("v.post_ln.weight") else None, proj)


_HF_BLOCK = {"ln1": "layer_norm1", "ln2": "layer_norm2", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
             "attn_v": "self_attn.v_proj", "attn_out": "self_attn.out_proj", "ffn_up": "mlp.fc1", "ffn_down": "mlp.fc2"}


def convert_vision_tower(src_dir: str, out_path: str) -> str:
    """Hugging Face LLaVA directory (``config.json`` with ``vision_config``, SafeTensors with ``vision_tower.*`` and
    ``multi_modal_projector.*``) → projector file."""
    with open(os.path.join(src_dir, "config.json")) as f:
        cfg = json.load(f)
    vc = cfg.get("vision_config") or cfg
    tensors: Dict[str, Tuple[SafeTensorsFile, str]] = {}
    for p in sorted(glob.glob(os.path.join(src_dir, "*.safetensors"))):
        st = SafeTensorsFile(p)
        for k in st.keys():
            tensors[k] = (st, k)

    def find(suffix: str):
        hits = [k for k in tensors if k.endswith(suffix)]
        if not hits:
            return None
        st, k = tensors[min(hits, key=len)]
        return st.tensor_f32(k)

    proj0 = find("multi_modal_projector.linear_1.weight")
    proj2 = find("multi_modal_projector.linear_2.weight")
    U, Fl = GGUFValueType.UINT32, GGUFValueType.FLOAT32
    w = GGUFWriter(out_path, arch="clip")
    w.add("clip.has_vision_encoder", True)
    w.add("clip.projector_type", "mlp")
    w.add("clip.vision.image_size", int(vc["image_size"]), U)
    w.add("clip.vision.patch_size", int(vc["patch_size"]), U)
    w.add("clip.vision.embedding_length", int(vc["hidden_size"]), U)
    w.add("clip.vision.feed_forward_length", int(vc["intermediate_size"]), U)
    w.add("clip.vision.block_count", int(vc["num_hidden_layers"]), U)
    w.add("clip.vision.attention.head_count", int(vc["num_attention_heads"]), U)
    w.add("clip.vision.attention.layer_norm_epsilon", float(vc.get("layer_norm_eps", 1e-5)), Fl)
    w.add("clip.vision.projection_dim", int(proj2.shape[0] if proj2 is not None else vc.get("projection_dim", 0)), U)
    w.add("clip.vision.image_mean", [float(x) for x in CLIP_MEAN])
    w.add("clip.vision.image_std", [float(x) for x in CLIP_STD])
    layer = cfg.get("vision_feature_layer", -2)
    w.add("clip.vision.feature_layer", int(layer if isinstance(layer, int) else layer[-1]), GGUFValueType.INT32)
    w.add("clip.use_gelu", str(vc.get("hidden_act", "quick_gelu")) == "gelu")

    def put(name: str, arr):
        if arr is None:
            raise ValueError(f"the checkpoint has no tensor for {name}")
        w.add_tensor(name, np.ascontiguousarray(arr, dtype=np.float32), arr.shape, "F32")

    put("v.patch_embd.weight", find("embeddings.patch_embedding.weight"))
    put("v.class_embd", find("embeddings.class_embedding"))
    put("v.position_embd.weight", find("embeddings.position_embedding.weight"))
    for half in ("weight", "bias"):
        put(f"v.pre_ln.{half}", find(f"pre_layrnorm.{half}"))  # (the misspelling is the checkpoint's own)
        post = find(f"post_layernorm.{half}")
        if post is not None:
            put(f"v.post_ln.{half}", post)
    for i in range(int(vc["num_hidden_layers"])):
        for gname, hname in _HF_BLOCK.items():
            for half in ("weight", "bias"):
                put(f"v.blk.{i}.{gname}.{half}", find(f"encoder.layers.{i}.{hname}.{half}"))
    if proj0 is not None:
        put("mm.0.weight", proj0)
        put("mm.0.bias", find("multi_modal_projector.linear_1.bias"))
        put("mm.2.weight", proj2)
        put("mm.2.bias", find("multi_modal_projector.linear_2.bias"))
    w.write()
    return out_path
