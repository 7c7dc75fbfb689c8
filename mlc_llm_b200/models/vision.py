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
        if config.get("model_type") in ("phi3_v", "phi3v"):
            # the checkpoint's own config: the parser fills in the tiling and the CLIP defaults
            from . import config as model_config  # pylint: disable=import-outside-toplevel

            return model_config.from_dict(config["model_type"], config).extra["vision"]
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
    if vision.get("kind") == "phi3v":
        pixels = hd_preprocess_pixels(arr, size, int(vision.get("hd_num", 4)))
        return pixels, hd_embed_size(pixels.shape[1] // size, pixels.shape[2] // size, size // int(vision["patch_size"]))
    pixels = preprocess_pixels(arr.unsqueeze(0), size)[0]
    return pixels, embed_size_of(vision)


def hd_target_shape(height: int, width: int, size: int, hd_num: int) -> Tuple[int, int, int]:
    """Phi-3-vision "HD transform" geometry: the largest ``scale`` with ``scale * ceil(scale / ratio) <=
    hd_num`` tiles, the resized extent ``(new_h, new_w)`` (long side = ``scale * size``) and the height
    after padding to whole tiles. A portrait image is handled transposed by the caller.
    Reference: ``cpp/support/vlm_utils.cc:12`` (``CalculateResizeShape`` / ``CalculatePadShape``)."""
    ratio = width / height
    scale = 1
    while scale * math.ceil(scale / ratio) <= hd_num:
        scale += 1
    scale -= 1
    new_w = scale * size
    new_h = int(new_w / ratio)
    padded_h = int(math.ceil(new_h / size) * size)
    return new_h, new_w, padded_h


def hd_preprocess_pixels(image: torch.Tensor, size: int, hd_num: int = 4) -> torch.Tensor:
    """``[3, H, W]`` values in 0..255 -> the padded high-definition image ``[3, h_crop * size,
    w_crop * size]``, normalised with the CLIP statistics: resize so the long side spans ``scale``
    tiles, pad the short side with white to whole tiles (centred). The tile grid is carried by the
    shape; the tower cuts the tiles and derives the global view itself."""
    _, h, w = image.shape
    transposed = w < h
    if transposed:
        image = image.transpose(1, 2)
        h, w = w, h
    new_h, new_w, padded_h = hd_target_shape(h, w, size, hd_num)
    x = F.interpolate(image.unsqueeze(0).float(), size=(max(new_h, 1), new_w), mode="bilinear",
                      align_corners=False)[0]
    top = (padded_h - new_h) // 2
    x = F.pad(x, (0, 0, top, padded_h - new_h - top), value=255.0)
    if transposed:
        x = x.transpose(1, 2)
    x = x / 255.0
    mean = torch.tensor(CLIP_MEAN, dtype=x.dtype).view(3, 1, 1)
    std = torch.tensor(CLIP_STD, dtype=x.dtype).view(3, 1, 1)
    return ((x - mean) / std).contiguous()


def hd_embed_size(h_crop: int, w_crop: int, side: int) -> int:
    """Prompt rows of one Phi-3-vision image: the tile grid's merged features with one separator per
    row, one separator between the two views, then the global view with its row separators
    (``side`` = patches per tile edge; 2x2 patches merge into one row entry)."""
    m = side // 2
    return (h_crop * m) * (w_crop * m + 1) + 1 + m * (m + 1)


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
        self.act_name = {"quick_gelu": "quick_gelu", "gelu": "gelu",
                         "gelu_pytorch_tanh": "gelu_tanh"}[vision.get("hidden_act", "quick_gelu")]
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
    @classmethod
    def projector_shapes(cls, vision: Dict[str, Any], text_hidden: int) -> Dict[str, tuple]:
        h, p = int(vision["hidden_size"]), cls.P
        return {p + "linear_1.weight": (text_hidden, h), p + "linear_1.bias": (text_hidden,),
                p + "linear_2.weight": (text_hidden, text_hidden), p + "linear_2.bias": (text_hidden,)}

    @classmethod
    def param_shapes(cls, vision: Dict[str, Any], text_hidden: int) -> Dict[str, tuple]:
        h, inter = int(vision["hidden_size"]), int(vision["intermediate_size"])
        patch, size = int(vision["patch_size"]), int(vision["image_size"])
        n_pos = (size // patch) ** 2 + 1
        v = cls.V
        shapes = {v + "embeddings.class_embedding": (h,),
                  v + "embeddings.patch_embedding.weight": (h, 3, patch, patch),
                  v + "embeddings.position_embedding.weight": (n_pos, h),
                  v + "pre_layrnorm.weight": (h,), v + "pre_layrnorm.bias": (h,),
                  v + "post_layernorm.weight": (h,), v + "post_layernorm.bias": (h,)}
        shapes.update(cls.projector_shapes(vision, text_hidden))
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

    @classmethod
    def random_params(cls, vision: Dict[str, Any], text_hidden: int, seed: int) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        out = {}
        for name, shape in cls.param_shapes(vision, text_hidden).items():
            if "norm" in name and name.endswith(".weight"):
                out[name] = torch.ones(shape)
            elif name.endswith(".bias"):
                out[name] = torch.zeros(shape)
            else:
                out[name] = torch.randn(shape, generator=g) * 0.02
        return out

    # ------------------------------------------------------------------ forward
    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        return ops.layernorm(x, self.t[name + ".weight"], self.t[name + ".bias"], self.eps)

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
            q = ops.linear(flat, self.lin[b + "self_attn.q_proj"]).view(n, -1, self.heads, d)
            k = ops.linear(flat, self.lin[b + "self_attn.k_proj"]).view(n, -1, self.heads, d)
            val = ops.linear(flat, self.lin[b + "self_attn.v_proj"]).view(n, -1, self.heads, d)
            ctx = ops.encoder_attention(q, k, val, scale=1.0 / math.sqrt(d)).to(self.dtype).reshape(-1, self.hidden)
            x = x + ops.linear(ctx, self.lin[b + "self_attn.out_proj"]).view(n, -1, self.hidden)
            h = self._ln(x, b + "layer_norm2").reshape(-1, self.hidden)
            h = ops.activation(ops.linear(h, self.lin[b + "mlp.fc1"]), self.act_name)
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


class Phi3VisionTower(VisionTower):
    """Phi-3-vision image embedding: CLIP features of a global view and of every tile of the padded
    high-definition image, 2x2 neighbouring patches concatenated on the channel axis, a learned
    separator row after every feature row (``sub_GN``) and between the two views (``glb_GN``), then a
    two-layer GELU projection into the language model's width.
    Reference: ``python/mlc_llm/model/phi3v/phi3v_image.py`` (``Phi3ImageEmbedding``: tiles first,
    then the separator, then the global view)."""

    V = "model.vision_embed_tokens.img_processor.vision_model."
    P = "model.vision_embed_tokens.img_projection."
    G = "model.vision_embed_tokens."

    @classmethod
    def projector_shapes(cls, vision: Dict[str, Any], text_hidden: int) -> Dict[str, tuple]:
        h4 = 4 * int(vision["hidden_size"])
        return {cls.P + "0.weight": (text_hidden, h4), cls.P + "0.bias": (text_hidden,),
                cls.P + "2.weight": (text_hidden, text_hidden), cls.P + "2.bias": (text_hidden,),
                cls.G + "glb_GN": (1, 1, h4), cls.G + "sub_GN": (1, 1, 1, h4)}

    def _merge_2x2(self, feats: torch.Tensor, h_crop: int, w_crop: int) -> torch.Tensor:
        """``[h_crop * w_crop, side * side, C]`` (tiles in row-major order) -> ``[h_crop * m, w_crop * m,
        4C]`` with ``m = side / 2``: each output entry is the 2x2 patch block (row-major) on the channel axis."""
        n, length, c = feats.shape
        side = int(math.isqrt(length))
        m = side // 2
        x = feats.view(n, m, 2, m, 2, c).permute(0, 1, 3, 2, 4, 5).reshape(n, m, m, 4 * c)
        x = x.view(h_crop, w_crop, m, m, 4 * c).permute(0, 2, 1, 3, 4)
        return x.reshape(h_crop * m, w_crop * m, 4 * c)

    def _with_row_separators(self, grid: torch.Tensor) -> torch.Tensor:
        sep = self.t[self.G + "sub_GN"].view(1, 1, -1).expand(grid.shape[0], 1, -1)
        return torch.cat([grid, sep], dim=1).reshape(-1, grid.shape[-1])

    def embed(self, pixels: torch.Tensor) -> torch.Tensor:
        """The padded high-definition image ``[3, h_crop * S, w_crop * S]`` -> prompt rows
        ``[hd_embed_size(h_crop, w_crop, S / patch), text_hidden]``."""
        s = self.size
        _, hh, ww = pixels.shape
        h_crop, w_crop = hh // s, ww // s
        x = pixels.to(self.device).float()
        global_view = F.interpolate(x.unsqueeze(0), size=(s, s), mode="bicubic", align_corners=False)
        tiles = x.reshape(3, h_crop, s, w_crop, s).permute(1, 3, 0, 2, 4).reshape(h_crop * w_crop, 3, s, s)
        feats = self.features(torch.cat([global_view, tiles], dim=0))[:, 1:]  # class token dropped
        glob = self._with_row_separators(self._merge_2x2(feats[:1], 1, 1))
        sub = self._with_row_separators(self._merge_2x2(feats[1:], h_crop, w_crop))
        rows = torch.cat([sub, self.t[self.G + "glb_GN"].view(1, -1), glob], dim=0).to(self.dtype)
        h = F.gelu(ops.linear(rows.contiguous(), self.lin[self.P + "0"]).float()).to(self.dtype)
        return ops.linear(h, self.lin[self.P + "2"])


def tower_class(vision: Dict[str, Any]):
    """The tower implementation a vision section asks for (``kind``: "llava" by default, "phi3v")."""
    return Phi3VisionTower if vision.get("kind") == "phi3v" else VisionTower


def load_hf_vision_params(path: str, vision: Dict[str, Any], text_hidden: int) -> Dict[str, torch.Tensor]:
    """Vision-tower and projector tensors of a HuggingFace LLaVA / Phi-3-vision checkpoint directory."""
    from ..loader.huggingface_loader import HFCheckpoint  # pylint: disable=import-outside-toplevel

    ckpt = HFCheckpoint(path)
    out = {}
    for name in tower_class(vision).param_shapes(vision, text_hidden):
        src = ckpt.resolve(name)
        if src is None:
            raise ValueError(f"checkpoint {path} has no tensor for {name}")
        out[name] = ckpt.get(src).clone()
    return out
