"""Request input data (reference: ``python/mlc_llm/serve/data.py`` / ``cpp/serve/data.h:37-251``)."""

from __future__ import annotations

import base64
import dataclasses
import io
from typing import List, Optional


class Data:
    """Base class of request inputs."""


class TextData(Data):
    def __init__(self, text: str):
        self.text = text

    def __repr__(self):
        return f"TextData({self.text!r})"


class TokenData(Data):
    def __init__(self, token_ids: List[int]):
        self.token_ids = list(token_ids)

    def __len__(self):
        return len(self.token_ids)


class ImageData(Data):
    """Pixel values plus the number of embedding rows the vision tower will produce."""

    def __init__(self, image, embed_size: int):
        self.image = image
        self.embed_size = embed_size

    def __len__(self):
        return self.embed_size

    @staticmethod
    def get_embed_size(config) -> int:
        """Prompt rows of one fixed-size (CLIP / LLaVA) image for this model's chat config."""
        from ..models.vision import embed_size_of, vision_dict  # pylint: disable=import-outside-toplevel

        return embed_size_of(vision_dict(config))

    @staticmethod
    def get_input_size(config) -> int:
        """Edge length, in pixels, of the square the vision tower reads."""
        from ..models.vision import vision_dict  # pylint: disable=import-outside-toplevel

        return int(vision_dict(config)["image_size"])

    @staticmethod
    def from_url(url: str, config) -> "ImageData":
        """Accepts ``data:image/...;base64,`` URLs and local file paths; pre-processing
        (resize / crop / normalise) is delegated to the model family's image processor."""
        from PIL import Image  # pylint: disable=import-outside-toplevel

        if url.startswith("data:"):
            raw = base64.b64decode(url.split(",", 1)[1])
            img = Image.open(io.BytesIO(raw)).convert("RGB")
        elif url.startswith("http"):
            import requests  # pylint: disable=import-outside-toplevel

            img = Image.open(io.BytesIO(requests.get(url, timeout=30).content)).convert("RGB")
        else:
            img = Image.open(url).convert("RGB")
        from ..models.vision import preprocess_image  # pylint: disable=import-outside-toplevel

        pixels, embed_size = preprocess_image(img, config)
        return ImageData(pixels, embed_size)


@dataclasses.dataclass
class SingleRequestStreamOutput:
    """What one choice of a request produced since the previous callback (reference:
    ``python/mlc_llm/serve/data.py:132``)."""

    delta_token_ids: List[int]
    delta_logprob_json_strs: Optional[List[str]]
    finish_reason: Optional[str]
    request_final_usage_json_str: Optional[str]
    extra_prefix_string: str


class RequestStreamOutput:
    """One engine callback item (mirrors the native ``RequestStreamOutput``)."""

    def __init__(self, d: dict):
        self.request_id: str = d["request_id"]
        self.group_delta_token_ids: List[List[int]] = d["group_delta_token_ids"]
        self.group_delta_logprob_json_strs: List[List[str]] = d["group_delta_logprob_json_strs"]
        self.group_finish_reason: List[Optional[str]] = d["group_finish_reason"]
        self.group_extra_prefix_string: List[str] = d["group_extra_prefix_string"]
        self.request_final_usage_json_str: Optional[str] = d["request_final_usage_json_str"]

    def unpack(self):
        """``(request_id, [SingleRequestStreamOutput per choice])``; the final item of a request carries
        only the usage string (reference: ``python/mlc_llm/serve/data.py:176``)."""
        if self.request_final_usage_json_str is not None:
            return self.request_id, [SingleRequestStreamOutput([], None, None, self.request_final_usage_json_str, "")]
        outs = []
        for i, ids in enumerate(self.group_delta_token_ids):
            lps = self.group_delta_logprob_json_strs[i] if i < len(self.group_delta_logprob_json_strs) else None
            outs.append(SingleRequestStreamOutput(
                list(ids), [str(s) for s in lps] if lps else None,
                self.group_finish_reason[i] if i < len(self.group_finish_reason) else None, None,
                self.group_extra_prefix_string[i] if i < len(self.group_extra_prefix_string) else ""))
        return self.request_id, outs
