"""Image inputs: CLIP vision tower, LLaVA projector and the image pre-processing in front of them.

Reference: ``python/mlc_llm/model/vision/clip_vision.py`` (CLIP ViT with pre-layernorm, quick-GELU MLP,
features taken from the second-to-last block), ``python/mlc_llm/model/vision/image_processing.py``
(resize to the shortest edge, centre crop, rescale by 1/255, normalise) and
``python/mlc_llm/model/llava/llava_model.py`` (``multi_modal_projector``: linear, GELU, linear; the
class token is dropped, so one image becomes ``(image_size / patch_size) ** 2`` embedding rows).

The tower runs once per image at request admission, far off the token loop, so it is written with
plain tensor ops (its matmuls go through ``ops.linear`` and therefore through this package's GEMM on
a GPU); parameters keep their HuggingFace names.
"""

from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def vision_dict(config: Any) -> Optional[Dict[str, Any]]:
    """The vision section of a model config (``ModelConfig.extra['vision']``, a chat-config dict with
    ``vision_config`` or the section itself); None for text-only models."""
    if config is None:
        return None
    extra = getattr(config, "extra", None)
    if isinstance(extra, dict) and "vision" in extra:
        return extra["vision"]
    if isinstance(config, dict):
        if isinstance(config.get("extra"), dict) and "vision" in config["extra"]:
            return config["extra"]["vision"]
        if "vision_config" in config:
            return config["vision_config"]
        if "model_config" in config and isinstance(config["model_config"], dict):
            return vision_dict(config["model_config"])
        if "image_size" in config and "patch_size" in config:
            return config
    return None


def embed_size_of(vision: Dict[str, Any]) -> int:
    side = int(vision["image_size"]) // int(vision["patch_size"])
    return side * side


def preprocess_image(img, config) -> Tuple[torch.Tensor, int]:
    """PIL image (RGB) -> normalised pixels ``[3, S, S]`` fp32 and the number of embedding rows the image
    will occupy in the prompt."""
    vision = vision_dict(config)
    if vision is None:
        raise ValueError("this model does not take image inputs")
    size = int(vision["image_size"])
    arr = torch.from_numpy(np.asarray(img.convert("RGB"), dtype=np.uint8).copy()).permute(2, 0, 1).float()
    pixels = preprocess_pixels(arr.unsqueeze(0), size)[0]
    return pixels, embed_size_of(vision)


def preprocess_pixels(image: torch.Tensor, size: int) -> torch.Tensor:
    """``[N, 3, H, W]`` values in 0..255 -> resize (shortest edge = ``size``, bilinear), centre crop to
    ``size`` x ``size``, rescale to 0..1, normalise with the CLIP statistics."""
    _, _, h, w = image.shape
    short, long = (w, h) if w <= h else (h, w)
    new_short, new_long = size, int(size * (long / short))
    nh, nw = (new_long, new_short) if w <= h else (new_short, new_long)
    x = F.interpolate(image.float(), size=(nh, nw), mode="bilinear", align_corners=False)
    top, left = (nh - size) // 2, (nw - size) // 2
    x = x[:, :, top: top + size, left: left + size] / 255.0
    mean = torch.tensor(CLIP_MEAN, dtype=x.dtype, device=x.device).view(1, 3, 1, 1)
    std = torch.tensor(CLIP_STD, dtype=x.dtype, device=x.device).view(1, 3, 1, 1)
    return (x - mean) / std


def _quick_gelu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(1.702 * x)


_ACT = {"quick_gelu": _quick_gelu, "gelu": F.gelu, "gelu_pytorch_tanh": lambda x: F.gelu(x, approximate="tanh")}


class VisionTower:
    """CLIP vision encoder + LLaVA projector; ``embed(pixels)`` returns the rows that stand in for the
    image inside the prompt, ``[embed_size, text_hidden]``."""

    V = "vision_tower.vision_model."
    P = "multi_modal_projector."

    def __init__(self, vision: Dict[str, Any], params: Dict[str, torch.Tensor], device: torch.device,
                 dtype: torch.dtype, feature_layer: int = -2, select: str = "default",
                 projector_act: str = "gelu"):
        self.cfg = vision
        self.device, self.dtype = device, dtype
        self.hidden = int(vision["hidden_size"])
        self.heads = int(vision["num_attention_heads"])
        self.layers = int(vision["num_hidden_layers"])
        self.patch = int(vision["patch_size"])
        self.size = int(vision["image_size"])
        self.eps = float(vision.get("layer_norm_eps", 1e-5))
        self.act = _ACT[vision.get("hidden_act", "quick_gelu")]
        self.proj_act = _ACT[projector_act]
        self.feature_layer = feature_layer
        self.select = select
        self.t: Dict[str, torch.Tensor] = {}
        self.lin: Dict[str, ops.LinearWeight] = {}
        for name, w in params.items():
            w = w.to(device=device, dtype=dtype)
            if name.endswith(".weight") and w.dim() == 2 and "embedding" not in name:
                self.lin[name[: -len(".weight")]] = ops.dense_weight(w.contiguous())
            else:
                self.t[name] = w
        for base, lw in self.lin.items():
            b = self.t.pop(base + ".bias", None)
            if b is not None:
                lw.bias = b.contiguous()

    # ------------------------------------------------------------------ parameters
    @staticmethod
    def param_shapes(vision: Dict[str, Any], text_hidden: int) -> Dict[str, tuple]:
        h, inter = int(vision["hidden_size"]), int(vision["intermediate_size"])
        patch, size = int(vision["patch_size"]), int(vision["image_size"])
        n_pos = (size // patch) ** 2 + 1
        v, p = VisionTower.V, VisionTower.P
        shapes = {v + "embeddings.class_embedding": (h,),
                  v + "embeddings.patch_embedding.weight": (h, 3, patch, patch),
                  v + "embeddings.position_embedding.weight": (n_pos, h),
                  v + "pre_layrnorm.weight": (h,), v + "pre_layrnorm.bias": (h,),
                  v + "post_layernorm.weight": (h,), v + "post_layernorm.bias": (h,),
                  p + "linear_1.weight": (text_hidden, h), p + "linear_1.bias": (text_hidden,),
                  p + "linear_2.weight": (text_hidden, text_hidden), p + "linear_2.bias": (text_hidden,)}
        for i in range(int(vision["num_hidden_layers"])):
            b = f"{v}encoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                shapes[b + f"self_attn.{n}.weight"] = (h, h)
                shapes[b + f"self_attn.{n}.bias"] = (h,)
            for n in ("layer_norm1", "layer_norm2"):
                shapes[b + n + ".weight"] = (h,)
                shapes[b + n + ".bias"] = (h,)
            shapes[b + "mlp.fc1.weight"] = (inter, h)
            shapes[b + "mlp.fc1.bias"] = (inter,)
            shapes[b + "mlp.fc2.weight"] = (h, inter)
            shapes[b + "mlp.fc2.bias"] = (h,)
        return shapes

    @staticmethod
    def random_params(vision: Dict[str, Any], text_hidden: int, seed: int) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        out = {}
        for name, shape in VisionTower.param_shapes(vision, text_hidden).items():
            if "norm" in name and name.endswith(".weight"):
                out[name] = torch.ones(shape)
            elif name.endswith(".bias"):
                out[name] = torch.zeros(shape)
            else:
                out[name] = torch.randn(shape, generator=g) * 0.02
        return out

    # ------------------------------------------------------------------ forward
    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return F.layer_norm(x.float(), (x.shape[-1],), self.t[name + ".weight"].float(),
                            self.t[name + ".bias"].float(), self.eps).to(x.dtype)

    def features(self, pixels: torch.Tensor) -> torch.Tensor:
        """``[N, 3, S, S]`` -> hidden states of the selected block, ``[N, 1 + patches, hidden]``."""
        v = self.V
        x = pixels.to(device=self.device, dtype=self.dtype)
        n = x.shape[0]
        # non-overlapping patches: the convolution is a matmul over unfolded patches
        w = self.t[v + "embeddings.patch_embedding.weight"]
        patches = F.unfold(x.float(), kernel_size=self.patch, stride=self.patch).transpose(1, 2)  # [N, P, 3*p*p]
        emb = (patches @ w.reshape(self.hidden, -1).float().t()).to(self.dtype)
        cls = self.t[v + "embeddings.class_embedding"].view(1, 1, -1).expand(n, 1, -1)
        x = torch.cat([cls, emb], dim=1) + self.t[v + "embeddings.position_embedding.weight"].unsqueeze(0)
        x = self._ln(x, v + "pre_layrnorm")
        last = self.layers + self.feature_layer + 1 if self.feature_layer < 0 else self.feature_layer
        d = self.hidden // self.heads
        for i in range(last):
            b = f"{v}encoder.layers.{i}."
            h = self._ln(x, b + "layer_norm1")
            flat = h.reshape(-1, self.hidden)
            q = ops.linear(flat, self.lin[b + "self_attn.q_proj"]).view(n, -1, self.heads, d).transpose(1, 2)
            k = ops.linear(flat, self.lin[b + "self_attn.k_proj"]).view(n, -1, self.heads, d).transpose(1, 2)
            val = ops.linear(flat, self.lin[b + "self_attn.v_proj"]).view(n, -1, self.heads, d).transpose(1, 2)
            att = torch.softmax((q.float() @ k.float().transpose(-1, -2)) / math.sqrt(d), dim=-1)
            ctx = (att @ val.float()).to(self.dtype).transpose(1, 2).reshape(-1, self.hidden)
            x = x + ops.linear(ctx, self.lin[b + "self_attn.out_proj"]).view(n, -1, self.hidden)
            h = self._ln(x, b + "layer_norm2").reshape(-1, self.hidden)
            h = self.act(ops.linear(h, self.lin[b + "mlp.fc1"]).float()).to(self.dtype)
            x = x + ops.linear(h, self.lin[b + "mlp.fc2"]).view(n, -1, self.hidden)
        return x

    def embed(self, pixels: torch.Tensor) -> torch.Tensor:
        """One image ``[3, S, S]`` (or a batch) -> ``[N * embed_size, text_hidden]`` prompt rows."""
        if pixels.dim() == 3:
            pixels = pixels.unsqueeze(0)
        f = self.features(pixels)
        if self.select == "default":
            f = f[:, 1:]  # drop the class token
        flat = f.reshape(-1, self.hidden)
        h = self.proj_act(ops.linear(flat, self.lin[self.P + "linear_1"]).float()).to(self.dtype)
        return ops.linear(h, self.lin[self.P + "linear_2"])


def load_hf_vision_params(path: str, vision: Dict[str, Any], text_hidden: int) -> Dict[str, torch.Tensor]:
    """Vision-tower and projector tensors of a HuggingFace LLaVA checkpoint directory."""
    from ..loader.huggingface_loader import HFCheckpoint  # pylint: disable=import-outside-toplevel

    ckpt = HFCheckpoint(path)
    out = {}
    for name in VisionTower.param_shapes(vision, text_hidden):
        src = ckpt.resolve(name)
        if src is None:
            raise ValueError(f"checkpoint {path} has no tensor for {name}")
        out[name] = ckpt.get(src).clone()
    return out
