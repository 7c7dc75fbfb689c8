"""Embedding inference for the ``/v1/embeddings`` endpoint (reference:
``python/mlc_llm/serve/embedding_engine.py:20-490``).

Two model kinds:

* encoder (BERT-style, ``models/bert.py``): ``[CLS] text [SEP]``, pooling ``cls`` (default) or ``mean``;
* decoder (Qwen3-Embedding style): the text (plus EOS) is prefilled through the regular paged decoder
  and the hidden state of the last token is the embedding (pooling ``last``; ``mean`` also supported).

Vectors are L2-normalised by default. Inference runs on one worker thread so the asyncio loop of
the server stays responsive.
"""

from __future__ import annotations

import asyncio
import concurrent.futures
import json
import math
import os
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import _core
from .. import quantization as Q
from ..models import config as model_config
from ..models import loader as model_loader
from ..models.transformer import BatchInfo, DecoderModel
from ..tokenizers import Tokenizer
from .engine_base import detect_device, resolve_model


class AsyncEmbeddingEngine:
    def __init__(self, model: str, model_lib: Optional[str] = None, device: Union[str, torch.device] = "auto", *,
                 pooling_strategy: Optional[str] = None, normalize: bool = True, max_batch_tokens: int = 8192):
        self.device = detect_device(device)
        self.model = model
        self.normalize = normalize
        self.max_batch_tokens = max_batch_tokens
        path = model if os.path.isdir(model) else None
        hf_cfg = {}
        if path and os.path.exists(os.path.join(path, "config.json")):
            with open(os.path.join(path, "config.json"), encoding="utf-8") as f:
                hf_cfg = json.load(f)
        self.model_type = "encoder" if hf_cfg.get("model_type") in ("bert", "roberta", "xlm-roberta") else "decoder"
        if self.model_type == "encoder":
            from ..models.bert import BertModel  # pylint: disable=import-outside-toplevel

            self.tokenizer = Tokenizer(path)
            self.encoder = BertModel.from_hf(path, self.device)
            self.cls_id, self.sep_id = self._special_ids(path)
            self.pad_id = int(hf_cfg.get("pad_token_id", 0))
            self.max_len = int(hf_cfg.get("max_position_embeddings", 512))
        else:
            info = resolve_model(model)
            chat = info.chat_config
            mc = dict(chat.get("model_config", {}))
            self.cfg = model_config.from_dict(chat["model_type"], mc)
            quant = Q.get(chat.get("quantization", "q0f16"))
            if info.random_seed is not None:
                store = model_loader.random_params(self.cfg, quant, info.random_seed, self.device)
            elif info.hf_weights:
                store = model_loader.load_hf_params(info.model_path, self.cfg, quant, self.device)
            else:
                store = model_loader.load_params(info.model_path, self.cfg, quant, self.device)
            self.decoder = DecoderModel(self.cfg, quant, store, self.device)
            self.pages = max(64, max_batch_tokens // 16 + 64)
            self.decoder.create_kv_cache(self.pages, 16)
            try:
                self.tokenizer = Tokenizer(info.model_path) if info.model_path else Tokenizer.synthetic(self.cfg.vocab_size)
            except ValueError:
                self.tokenizer = Tokenizer.synthetic(self.cfg.vocab_size)
            eos = chat.get("eos_token_id")
            self.eos_id = eos[0] if isinstance(eos, list) and eos else eos
            self.max_len = int(self.cfg.context_window_size)
        self.pooling_strategy = pooling_strategy or ("cls" if self.model_type == "encoder" else "last")
        if self.pooling_strategy not in ("cls", "mean", "last"):
            raise ValueError(f"unknown pooling strategy {self.pooling_strategy}")
        self._executor = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="embedding")
        self._terminated = False

    def _special_ids(self, path: str) -> Tuple[Optional[int], Optional[int]]:
        cls_id = sep_id = None
        cfg_path = os.path.join(path, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path, encoding="utf-8") as f:
                tc = json.load(f)
            for tid, info in (tc.get("added_tokens_decoder") or {}).items():
                if info.get("content") == tc.get("cls_token"):
                    cls_id = int(tid)
                if info.get("content") == tc.get("sep_token"):
                    sep_id = int(tid)
            if cls_id is None and tc.get("cls_token"):
                cls_id = self.tokenizer.token_to_id(tc["cls_token"])
            if sep_id is None and tc.get("sep_token"):
                sep_id = self.tokenizer.token_to_id(tc["sep_token"])
        return (cls_id if cls_id is not None and cls_id >= 0 else None,
                sep_id if sep_id is not None and sep_id >= 0 else None)

    # ------------------------------------------------------------------ public API
    async def async_embed(self, inputs: Sequence[Union[str, List[int]]]) -> Tuple[List[List[float]], int]:
        """``embed`` on the engine's worker thread, so the event loop stays free
        (reference: ``serve/embedding_engine.py:184``)."""
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(self._executor, self.embed, list(inputs))

    def embed_sync(self, inputs: Sequence[Union[str, List[int]]]) -> Tuple[List[List[float]], int]:
        return self.embed(inputs)

    def embed(self, inputs: Sequence[Union[str, List[int]]]) -> Tuple[List[List[float]], int]:
        """Embedding vectors (L2-normalised unless configured otherwise) and the number of input tokens;
        synchronous (reference: ``serve/embedding_engine.py:165``)."""
        ids = [list(x) if not isinstance(x, str) else self.tokenizer.encode(x) for x in inputs]
        if self.model_type == "encoder":
            vecs = self._embed_encoder(ids)
        else:
            vecs = self._embed_decoder(ids)
        if self.normalize:
            vecs = torch.nn.functional.normalize(vecs.float(), dim=-1)
        total = sum(len(x) for x in ids)
        return vecs.float().cpu().tolist(), total

    @staticmethod
    def truncate(vec: List[float], dimensions: int) -> List[float]:
        """Matryoshka-style truncation followed by re-normalisation."""
        v = vec[:dimensions]
        n = math.sqrt(sum(x * x for x in v)) or 1.0
        return [x / n for x in v]

    def terminate(self) -> None:
        if not self._terminated:
            self._terminated = True
            self._executor.shutdown(wait=True)

    # ------------------------------------------------------------------ model paths
    def _embed_encoder(self, ids: List[List[int]]) -> torch.Tensor:
        seqs = []
        for x in ids:
            x = x[: self.max_len - 2]
            if self.cls_id is not None and (not x or x[0] != self.cls_id):
                x = [self.cls_id] + x
            if self.sep_id is not None and (not x or x[-1] != self.sep_id):
                x = x + [self.sep_id]
            seqs.append(x)
        width = max(len(x) for x in seqs)
        toks = torch.full((len(seqs), width), self.pad_id, dtype=torch.long)
        mask = torch.zeros(len(seqs), width, dtype=torch.long)
        for i, x in enumerate(seqs):
            toks[i, : len(x)] = torch.tensor(x)
            mask[i, : len(x)] = 1
        h = self.encoder.forward(toks.to(self.device), mask.to(self.device)).float()
        m = mask.to(self.device).unsqueeze(-1).float()
        if self.pooling_strategy == "cls":
            return h[:, 0]
        if self.pooling_strategy == "mean":
            return (h * m).sum(1) / m.sum(1).clamp_min(1)
        last = mask.sum(1).to(self.device) - 1
        return h[torch.arange(len(seqs), device=self.device), last]

    def _embed_decoder(self, ids: List[List[int]]) -> torch.Tensor:
        out = []
        batch: List[List[int]] = []
        used = 0
        for x in ids:
            x = list(x[: self.max_len - 1])
            if self.eos_id is not None and (not x or x[-1] != self.eos_id):
                x.append(int(self.eos_id))
            if batch and used + len(x) > self.max_batch_tokens:
                out.append(self._decoder_batch(batch))
                batch, used = [], 0
            batch.append(x)
            used += len(x)
        if batch:
            out.append(self._decoder_batch(batch))
        return torch.cat(out, 0)

    def _decoder_batch(self, seqs: List[List[int]]) -> torch.Tensor:
        kv = _core.KVManager(self.pages, 16, len(seqs) + 1)
        for i in range(len(seqs)):
            kv.add_sequence(i)
        lens = [len(x) for x in seqs]
        plan = kv.begin_forward(list(range(len(seqs))), lens)
        t = lambda k: torch.from_numpy(np.asarray(plan[k])).to(torch.int32).to(self.device)
        b = BatchInfo(positions=t("positions"), slots=t("slots"), q_seq=t("q_seq"), q_kvlen=t("q_kvlen"),
                      page_indptr=t("page_indptr"), page_indices=t("page_indices"), num_tokens=sum(lens))
        toks = torch.tensor([tok for x in seqs for tok in x], dtype=torch.int32, device=self.device)
        m = self.decoder
        h = m.forward(m.embed(toks), b)
        normed = getattr(m, "_final_normed", None)
        h = normed if normed is not None else m._norm(h, "model.norm")  # pylint: disable=protected-access
        m._final_normed = None  # pylint: disable=protected-access
        ends = np.cumsum(lens)
        if self.pooling_strategy == "mean":
            return torch.stack([h[e - n: e].float().mean(0) for e, n in zip(ends, lens)])
        idx = torch.tensor(ends - 1, device=self.device)
        return h[idx].float()
