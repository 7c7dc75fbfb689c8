"""Shared machinery of the Python engines: model discovery, runtime construction (weights, KV
cache, executor, native engine), request -> prompt conversion and stream-output -> OpenAI response
conversion.

Reference: ``python/mlc_llm/serve/engine_base.py`` (:62-99 config checks, :119-181 model argument
processing, :556-684 engine construction, :687-887 request / response conversion, :1154-1213
function-call parsing, :242-270 Prometheus text).
"""

from __future__ import annotations

import ast
import dataclasses
import json
import os
import threading
import urllib.parse
import uuid
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import _core
from .. import quantization as Q
from ..conversation_template import ConvTemplateRegistry
from ..models import config as model_config
from ..models import loader as model_loader
from ..models.presets import MODEL_PRESETS
from ..models.transformer import DecoderModel
from ..protocol import openai_api_protocol as openai
from ..protocol.conversation_protocol import Conversation
from ..protocol.error_protocol import BadRequestError
from ..protocol.mlc_chat_config import MLC_CHAT_SYSTEM_DEFAULT
from ..tokenizers import Tokenizer
from . import data
from .config import EngineConfig
from .executor import ModelExecutor


# ------------------------------------------------------------------------------ model discovery
@dataclasses.dataclass
class ModelInfo:
    """A model argument resolved to its configuration and weight source."""

    model: str
    model_path: Optional[str]
    chat_config: Dict[str, Any]
    random_seed: Optional[int] = None  # set for "random://" models
    hf_weights: bool = False  # model_path is an unconverted HuggingFace checkpoint


def _random_model_chat_config(spec: str) -> Tuple[Dict[str, Any], int]:
    """``random://<preset>?quant=q4f16_1&seed=0&k=v`` -> a synthetic mlc-chat-config."""
    parsed = urllib.parse.urlparse(spec)
    preset = parsed.netloc or parsed.path.strip("/")
    if preset not in MODEL_PRESETS:
        raise ValueError(f"unknown preset {preset!r}; known: {sorted(MODEL_PRESETS)}")
    args = dict(urllib.parse.parse_qsl(parsed.query))
    quant = args.pop("quant", "q0f16")
    seed = int(args.pop("seed", 0))
    hf = dict(MODEL_PRESETS[preset])
    for k, v in args.items():
        try:
            hf[k] = json.loads(v)
        except json.JSONDecodeError:
            hf[k] = v
    mcfg = model_config.from_dict(hf["model_type"], hf)
    conv = ConvTemplateRegistry.get_conv_template(args.get("conv_template", "LM"))
    chat = {
        "version": "0.1.0", "model_type": hf["model_type"], "quantization": quant,
        "model_config": {**hf, **{k: v for k, v in mcfg.asdict().items() if k not in hf}},
        "vocab_size": mcfg.vocab_size, "context_window_size": mcfg.context_window_size,
        "sliding_window_size": mcfg.sliding_window_size, "prefill_chunk_size": mcfg.prefill_chunk_size,
        "attention_sink_size": mcfg.attention_sink_size,
        "tensor_parallel_shards": mcfg.tensor_parallel_shards,
        "pipeline_parallel_stages": mcfg.pipeline_parallel_stages,
        "temperature": 1.0, "top_p": 1.0, "presence_penalty": 0.0, "frequency_penalty": 0.0,
        "repetition_penalty": 1.0, "tokenizer_files": [], "tokenizer_info": {},
        "conv_template": conv.to_json_dict(), "pad_token_id": 0, "bos_token_id": 1,
        "eos_token_id": [2], "model_task": "chat",
    }
    return chat, seed


def resolve_model(model: str) -> ModelInfo:
    """Accepts a converted-model directory, its ``mlc-chat-config.json``, or ``random://preset``."""
    if model.startswith("random://"):
        chat, seed = _random_model_chat_config(model)
        return ModelInfo(model, None, chat, seed)
    if model.startswith("HF://") or model.startswith("https://"):
        from ..support.download_cache import get_or_download_model  # pylint: disable=import-outside-toplevel

        model_path = str(get_or_download_model(model))
    else:
        model_path = model
    if os.path.isfile(model_path):
        model_path = os.path.dirname(model_path)
    cfg_path = os.path.join(model_path, "mlc-chat-config.json")
    if not os.path.exists(cfg_path) and os.path.exists(os.path.join(model_path, "config.json")):
        return _resolve_hf_checkpoint(model, model_path)
    if not os.path.exists(cfg_path):
        raise FileNotFoundError(f"Cannot find mlc-chat-config.json under {model_path}")
    with open(cfg_path, encoding="utf-8") as f:
        chat = json.load(f)
    for k, v in MLC_CHAT_SYSTEM_DEFAULT.items():
        chat.setdefault(k, v)
    return ModelInfo(model, model_path, chat)


_DEFAULT_CONV = {"llama": "llama-2", "mistral": "mistral_default", "mixtral": "mistral_default",
                 "qwen2": "qwen2", "qwen3": "qwen3", "qwen2_moe": "qwen2", "qwen3_moe": "qwen3",
                 "gemma": "gemma_instruction", "gemma2": "gemma_instruction", "gemma3": "gemma3_instruction",
                 "phi3": "phi-3", "phi": "phi-2", "gpt2": "gpt2", "gpt_bigcode": "gpt_bigcode"}


def _resolve_hf_checkpoint(model: str, model_path: str) -> ModelInfo:
    """Serve an unconverted HuggingFace directory: the chat config is generated in memory
    (``gen_config`` defaults; quantisation from ``MLC_JIT_QUANTIZATION`` or the checkpoint dtype) and
    weights are quantised while loading — the counterpart of the reference's JIT path
    (``serve/engine_base.py:155-175``, ``interface/jit.py``)."""
    import tempfile  # pylint: disable=import-outside-toplevel

    from ..interface.gen_config import gen_config  # pylint: disable=import-outside-toplevel

    with open(os.path.join(model_path, "config.json"), encoding="utf-8") as f:
        hf = json.load(f)
    dtype = str(hf.get("torch_dtype", hf.get("dtype", "float16")))
    quant = os.environ.get("MLC_JIT_QUANTIZATION") or {"bfloat16": "q0bf16", "float32": "q0f32"}.get(dtype, "q0f16")
    mt = hf.get("model_type", "llama")
    conv = os.environ.get("MLC_JIT_CONV_TEMPLATE") or _DEFAULT_CONV.get(mt, "LM")
    if "llama" == mt and int(hf.get("vocab_size", 0)) > 100000:
        conv = "llama-3"
    with tempfile.TemporaryDirectory() as tmp:
        path = gen_config(model_path, "auto", quant, conv, None, None, None, None, None, None, None, 128, tmp)
        with open(path, encoding="utf-8") as f:
            chat = json.load(f)
    for k, v in MLC_CHAT_SYSTEM_DEFAULT.items():
        chat.setdefault(k, v)
    return ModelInfo(model, model_path, chat, None, True)


def conversation_of(chat_config: Dict[str, Any]) -> Conversation:
    conv = chat_config.get("conv_template", "LM")
    if isinstance(conv, str):
        tpl = ConvTemplateRegistry.get_conv_template(conv)
        if tpl is None:
            raise ValueError(f"Unknown conversation template {conv}")
        return tpl
    return Conversation.from_json_dict(conv)


def detect_device(device: Union[str, torch.device]) -> torch.device:
    if isinstance(device, torch.device):
        return device
    if device in ("auto", None):
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
    if device.startswith("cuda") and ":" not in device and torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device(device)


# ------------------------------------------------------------------------------ grammar backend
class XGrammarBackend:
    """JSON-mode constrained decoding over the ``xgrammar`` package (the reference links the same
    library in C++: ``cpp/serve/engine.cc:471-473``, ``request_state.cc:22-83``)."""

    def __init__(self, tokenizer: Tokenizer, vocab_size: int):
        import xgrammar as xgr  # pylint: disable=import-outside-toplevel

        self.xgr = xgr
        table = tokenizer.post_processed_token_table()
        info = xgr.TokenizerInfo(table, vocab_type=xgr.VocabType.RAW, vocab_size=vocab_size)
        self.compiler = xgr.GrammarCompiler(info)
        self.vocab_size = vocab_size
        self.matchers: Dict[int, Any] = {}
        self._next = 0

    def create(self, response_format_json: str) -> int:
        rf = json.loads(response_format_json)
        schema = rf.get("schema")
        compiled = (self.compiler.compile_json_schema(schema) if schema
                    else self.compiler.compile_builtin_json_grammar())
        h = self._next
        self._next += 1
        self.matchers[h] = self.xgr.GrammarMatcher(compiled, max_rollback_tokens=10)
        return h

    def release(self, h: int) -> None:
        self.matchers.pop(h, None)

    def next_token_bitmask(self, h: int):
        bm = self.xgr.allocate_token_bitmask(1, self.vocab_size)
        self.matchers[h].fill_next_token_bitmask(bm, 0)
        return bm.numpy().reshape(-1).astype(np.int32)

    def accept_token(self, h: int, token: int) -> bool:
        return bool(self.matchers[h].accept_token(int(token)))

    def rollback(self, h: int, n: int) -> None:
        self.matchers[h].rollback(n)

    def is_terminated(self, h: int) -> bool:
        return bool(self.matchers[h].is_terminated())

    def find_jump_forward_string(self, h: int) -> str:
        return self.matchers[h].find_jump_forward_string()


# ------------------------------------------------------------------------------ runtime
class EngineRuntime:
    """Everything below the native engine for one process: models, KV caches, executor, tokenizer.

    ``comm`` is the tensor-parallel communicator of this process (``parallel.Communicator``) or
    None. Only rank 0 builds a native engine; the other ranks run ``parallel.worker_loop``.
    """

    def __init__(self, engine_config: EngineConfig, device: Union[str, torch.device] = "auto",
                 comm=None, trace_recorder=None):
        self.device = detect_device(device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.comm = comm
        self.trace = trace_recorder
        cfg = engine_config
        if cfg.kv_cache_page_size != 16:
            raise ValueError("KV cache page size other than 16 is not supported.")
        self.is_mock = cfg.model_lib is not None and cfg.model_lib.startswith("mock://")
        self.models_info: List[ModelInfo] = [resolve_model(cfg.model)]
        for extra in cfg.additional_models:
            self.models_info.append(resolve_model(extra if isinstance(extra, str) else extra[0]))
        main = self.models_info[0]
        self.chat_config = main.chat_config
        self.conv_template = conversation_of(main.chat_config)
        self.tokenizer = self._make_tokenizer(main)
        self.models: List[DecoderModel] = []
        self.executor: Optional[ModelExecutor] = None
        self.grammar = None
        self.engine_config = cfg
        self.complete_config_json = cfg.asjson()
        self.num_pages: List[int] = []
        if not self.is_mock:
            self._build_models()

    # ---------------------------------------------------------------- pieces
    def _make_tokenizer(self, info: ModelInfo) -> Tokenizer:
        if info.model_path is not None:
            try:
                return Tokenizer(info.model_path)
            except ValueError:
                pass
        return Tokenizer.synthetic(int(info.chat_config["vocab_size"]))

    def _model_config(self, info: ModelInfo) -> model_config.ModelConfig:
        chat = info.chat_config
        mc = dict(chat.get("model_config", {}))
        for k in ("context_window_size", "prefill_chunk_size", "sliding_window_size",
                  "attention_sink_size", "tensor_parallel_shards", "pipeline_parallel_stages"):
            if k in chat and chat[k] is not None and k not in mc:
                mc[k] = chat[k]
        cfg = self.engine_config
        if cfg.tensor_parallel_shards:
            mc["tensor_parallel_shards"] = cfg.tensor_parallel_shards
        if cfg.pipeline_parallel_stages:
            mc["pipeline_parallel_stages"] = cfg.pipeline_parallel_stages
        return model_config.from_dict(chat["model_type"], mc)

    def _attach_vision_tower(self, model: DecoderModel, info: ModelInfo, mcfg) -> None:
        """Image inputs: the CLIP tower + projector produce the prompt rows of an image
        (``model.image_embed(pixels)``; reference: ``cpp/serve/model.cc`` ``ImageEmbed``)."""
        from ..models import vision as V  # pylint: disable=import-outside-toplevel

        vis = mcfg.extra["vision"]
        tower_cls = V.tower_class(vis)
        if info.random_seed is not None:
            params = tower_cls.random_params(vis, mcfg.hidden_size, info.random_seed + 101)
        elif info.hf_weights:
            params = V.load_hf_vision_params(info.model_path, vis, mcfg.hidden_size)
        else:
            from ..loader.tensor_cache import TensorCache  # pylint: disable=import-outside-toplevel

            cache = TensorCache(info.model_path)
            params = {n: cache.get(n) for n in tower_cls.param_shapes(vis, mcfg.hidden_size)}
        dtype = model.dtype if self.device.type == "cuda" else torch.float32
        tower = tower_cls(vis, params, self.device, dtype,
                              feature_layer=int(mcfg.extra.get("vision_feature_layer", -2)),
                              select=mcfg.extra.get("vision_feature_select_strategy", "default"),
                              projector_act=mcfg.extra.get("projector_hidden_act", "gelu"))
        model.vision_tower = tower
        model.image_embed = lambda pixels: tower.embed(pixels).to(model.dtype)

    def _build_models(self) -> None:
        cfg = self.engine_config
        comm = self.comm
        tp = comm.tp_size if comm is not None else 1
        tp_rank = comm.tp_rank if comm is not None else 0
        pp = comm.pp_size if comm is not None else 1
        pp_rank = comm.pp_rank if comm is not None else 0
        infos = []
        for mi, info in enumerate(self.models_info):
            mcfg = self._model_config(info)
            mcfg.tensor_parallel_shards = tp
            mcfg.pipeline_parallel_stages = pp if mi == 0 else 1
            quant = Q.get(info.chat_config.get("quantization", "q0f16"))
            if self.device.type == "cpu" and quant.torch_dtype != torch.float32 and quant.kind == "no-quant":
                pass  # half precision on CPU is slow but correct
            part = model_loader.layer_partition(mcfg)
            layers = range(part[pp_rank], part[pp_rank + 1]) if mi == 0 else range(mcfg.num_hidden_layers)
            if info.random_seed is not None:
                store = model_loader.random_params(mcfg, quant, info.random_seed, self.device, tp, tp_rank, layers)
            elif info.hf_weights:
                store = model_loader.load_hf_params(info.model_path, mcfg, quant, self.device, tp, tp_rank, layers)
            else:
                store = model_loader.load_params(info.model_path, mcfg, quant, self.device, tp, tp_rank, layers)
            if mcfg.extra.get("rwkv"):
                from ..models.rwkv import RwkvModel  # pylint: disable=import-outside-toplevel

                if pp > 1 or len(self.models_info) > 1:
                    raise ValueError("recurrent-state models run without pipeline stages and without a draft model")
                model = RwkvModel(mcfg, quant, store, self.device, comm if tp > 1 else None, layers)
                cfg.prefix_cache_mode = "disable"  # a recurrent state cannot be shared or rolled back
                cfg.kv_state_kind = "rnn_state"
            elif mcfg.extra.get("gdn"):
                from ..models.qwen35 import Qwen35Model  # pylint: disable=import-outside-toplevel

                if pp > 1 or len(self.models_info) > 1:
                    raise ValueError("hybrid recurrent-state models run without pipeline stages and without a "
                                     "draft model")
                model = Qwen35Model(mcfg, quant, store, self.device, comm if tp > 1 else None, layers)
                cfg.prefix_cache_mode = "disable"  # the recurrent half of the state cannot be shared or rolled back
                cfg.kv_state_kind = "hybrid"
            else:
                model = DecoderModel(mcfg, quant, store, self.device, comm if tp > 1 else None, layers)
            if mi == 0 and mcfg.extra.get("vision"):
                self._attach_vision_tower(model, info, mcfg)
            self.models.append(model)
            infos.append({
                "params_bytes": store.nbytes(), "num_layers": mcfg.num_hidden_layers,
                "num_qo_heads": model.hq, "num_kv_heads": getattr(model, "cache_kv_heads", model.hkv),
                "head_dim": getattr(model, "cache_head_dim", mcfg.head_dim),
                "vocab_size": mcfg.vocab_size, "context_window_size": mcfg.context_window_size,
                "sliding_window_size": mcfg.sliding_window_size,
                "prefill_chunk_size": mcfg.prefill_chunk_size, "max_batch_size": mcfg.max_batch_size,
                "pipeline_parallel_stages": mcfg.pipeline_parallel_stages,
                "kv_bytes_per_element": 4 if model.kv_dtype == torch.float32 else 2,
                "hidden_size": mcfg.hidden_size,
                "rnn_state_bytes_per_sequence": int(model.state_bytes_per_sequence())
                if hasattr(model, "state_bytes_per_sequence") else 0,
            })
        if self.device.type == "cuda":
            total = torch.cuda.get_device_properties(self.device).total_memory
        else:
            import psutil  # pylint: disable=import-outside-toplevel

            total = min(psutil.virtual_memory().available, 16 << 30)
        ec = json.loads(cfg.asjson())
        ec.setdefault("mode", "local")
        if ec.get("speculative_mode") == "medusa" and len(self.models) > 1 and self.models[1].cfg.extra.get("medusa"):
            # one draft token per Medusa head
            heads = int(self.models[1].cfg.extra["medusa"]["num_heads"])
            ec["spec_draft_length"] = min(int(ec.get("spec_draft_length") or heads), heads)
        res = _core.infer_capacity(json.dumps(ec), infos, int(total))
        if comm is not None and comm.world_size > 1:
            res = comm.agree_on_capacity(res)
        self.complete_config_json = res["config_json"]
        self.capacity_report = res["report"]
        n_pages = int(res["num_pages"])
        for m in self.models:
            m.create_kv_cache(n_pages, 16)
            self.num_pages.append(n_pages)
        full = json.loads(self.complete_config_json)
        self.fused_tp = False
        # MLCB_FUSED_TP: "1" = always, "0" = never, default "auto" = where the fused kernels, replayed
        # from CUDA graphs, measured above the NCCL path (2, 4 and 8 ranks).
        fused_mode = os.environ.get("MLCB_FUSED_TP", "auto")
        use_fused = fused_mode == "1" or (fused_mode == "auto" and tp in (2, 4, 8))
        # "1" on a single GPU runs the same kernels with one rank (peer tables point at local memory)
        for m in self.models:
            if m.cfg.expert_parallel and m.cfg.num_experts > 0 and tp > 1 and self.device.type == "cuda":
                from ..parallel.expert import ExpertParallel  # pylint: disable=import-outside-toplevel

                max_tokens = max(int(full.get("prefill_chunk_size") or 2048),
                                 int(full["max_num_sequence"]) * ((full.get("spec_draft_length") or 0) + 1))
                m.ep = ExpertParallel(m.cfg.num_experts, m.cfg.num_experts_per_tok, m.cfg.hidden_size, m.dtype,
                                      max_tokens, self.device, group=comm.tp_group, world_size=tp)
        if (tp > 1 or fused_mode == "1") and self.device.type == "cuda" and use_fused:
            # fused GEMM+collective kernels over symmetric peer buffers (main model only)
            from ..parallel.fused import FusedCollectives  # pylint: disable=import-outside-toplevel

            main_model = self.models[0]
            if main_model.cfg.norm_type == "rms" and main_model.dtype in (torch.float16, torch.bfloat16):
                max_tokens = max(int(full.get("prefill_chunk_size") or 2048),
                                 int(full["max_num_sequence"]) * ((full.get("spec_draft_length") or 0) + 1))
                fused = FusedCollectives(main_model.cfg.hidden_size, main_model.dtype, max_tokens, self.device,
                                         group=comm.tp_group if tp > 1 else None, world_size=tp)
                self.fused_tp = main_model.enable_fused(fused)
        slots = int(full["max_num_sequence"]) * 2 * ((full.get("spec_draft_length") or 4) + 1) \
            if full.get("speculative_mode", "disable") != "disable" else 0
        self.executor = ModelExecutor(self.models, self.device, comm, max_draft_slots=slots)
        try:
            self.grammar = XGrammarBackend(self.tokenizer, int(self.models[0].cfg.vocab_size))
        except Exception:  # pylint: disable=broad-except
            self.grammar = None  # JSON mode unavailable; requests asking for it are rejected upstream

    def eos_token_ids(self) -> List[int]:
        ids = list(self.conv_template.stop_token_ids or [])
        eos = self.chat_config.get("eos_token_id")
        if isinstance(eos, int):
            ids.append(eos)
        elif isinstance(eos, list):
            ids.extend(int(e) for e in eos)
        return sorted(set(ids))

    def make_core_engine(self, engine_config_json: Optional[str] = None, callback=None):
        """Builds the native engine (rank 0 only)."""
        cfg_json = engine_config_json or self.complete_config_json
        if self.is_mock:
            return _core.Engine.create_mock_echo(cfg_json, json.dumps(self.chat_config),
                                                 self.tokenizer.handle, callback)
        infos = []
        for info, model, pages in zip(self.models_info, self.models, self.num_pages):
            infos.append({"vocab_size": int(model.cfg.vocab_size), "num_pages": pages,
                          "eos_token_ids": self.eos_token_ids(),
                          "model_config_json": json.dumps(info.chat_config)})
        return _core.Engine.create(self.complete_config_json, infos, self.executor,
                                   self.tokenizer.handle, self.grammar, self.trace, callback)


# ------------------------------------------------------------------------------ request conversion
def get_generation_config(request: Union[openai.CompletionRequest, openai.ChatCompletionRequest],
                          extra_stop_token_ids: Optional[List[int]] = None,
                          extra_stop_str: Optional[List[str]] = None) -> Dict[str, Any]:
    """The JSON dict handed to the native ``GenerationConfig`` parser."""
    kwargs = openai.openai_api_get_generation_config(request)
    out: Dict[str, Any] = {}
    for k, v in kwargs.items():
        if v is None:
            continue
        if k == "response_format":
            out[k] = {"type": v.type, **({"schema": v.json_schema} if v.json_schema else {})}
        elif k == "debug_config":
            out[k] = v.model_dump(exclude_none=True)
        elif k == "logit_bias":
            out[k] = {str(t): b for t, b in v.items()}
        else:
            out[k] = v
    stops = list(out.get("stop_strs", []))
    for s in extra_stop_str or []:
        if s and s not in stops:
            stops.append(s)
    out["stop_strs"] = stops
    out["stop_token_ids"] = sorted(set(extra_stop_token_ids or []))
    return out


def process_chat_completion_request(request: openai.ChatCompletionRequest, request_id: str,
                                    runtime: EngineRuntime, max_input_len: int
                                    ) -> Tuple[List[Any], Dict[str, Any], bool, int]:
    """Apply the conversation template and tokenise. Returns (inputs, generation config dict,
    use_function_calling, prompt length)."""
    request.check_message_validity()
    conv = runtime.conv_template.model_copy(deep=True)
    request.check_function_call_usage(conv)
    for message in request.messages:
        role, content = message.role, message.content
        if role == "system":
            assert isinstance(content, str)
            conv.system_message = content if content is not None else ""
            continue
        conv.messages.append((role, content))
    conv.messages.append(("assistant", None))
    prompts = conv.as_prompt(runtime.chat_config.get("model_config"))
    inputs: List[Any] = []
    prefix = list(conv.system_prefix_token_ids or [])
    for i, p in enumerate(prompts):
        if isinstance(p, str):
            ids = runtime.tokenizer.encode(p)
            if i == 0 and prefix:
                ids = prefix + ids
            inputs.append(np.asarray(ids, dtype=np.int32))
        else:
            inputs.append(p)
    prompt_len = sum(len(x) for x in inputs)
    gen = get_generation_config(request, conv.stop_token_ids, conv.stop_str)
    if prompt_len > max_input_len:
        raise BadRequestError(f"Request prompt has {prompt_len} tokens in total, larger than the "
                              f"model input length limit {max_input_len}.")
    return inputs, gen, conv.use_function_calling, prompt_len


def process_completion_request(request: openai.CompletionRequest, request_id: str,
                               runtime: EngineRuntime, max_input_len: int
                               ) -> Tuple[List[Any], Dict[str, Any], int, Optional[str]]:
    """Returns (inputs, generation config dict, prompt length, echo text)."""
    prompt = request.prompt
    if isinstance(prompt, str):
        ids = runtime.tokenizer.encode(prompt)
        prefix = list(runtime.conv_template.system_prefix_token_ids or [])
        ids = prefix + ids
    else:
        ids = list(prompt)
    if len(ids) > max_input_len:
        raise BadRequestError(f"Request prompt has {len(ids)} tokens in total, larger than the model "
                              f"input length limit {max_input_len}.")
    gen = get_generation_config(request, runtime.conv_template.stop_token_ids, [])
    echo_text = None
    if request.echo:
        echo_text = prompt if isinstance(prompt, str) else runtime.tokenizer.decode(ids)
    return [np.asarray(ids, dtype=np.int32)], gen, len(ids), echo_text


def create_request_id(prefix: str, user: Optional[str]) -> str:
    return user if user is not None else f"{prefix}-{uuid.uuid4().hex}"


# ------------------------------------------------------------------------------ response helpers
def parse_logprobs(json_strs: Sequence[str]) -> Optional[openai.LogProbs]:
    if not json_strs:
        return None
    content = []
    for s in json_strs:
        d = json.loads(s)
        content.append(openai.LogProbsContent(
            token=d["token"], logprob=d["logprob"], bytes=d.get("bytes"),
            top_logprobs=[openai.TopLogProbs(token=t["token"], logprob=t["logprob"], bytes=t.get("bytes"))
                          for t in d.get("top_logprobs", [])]))
    return openai.LogProbs(content=content)


def parse_completion_logprobs(json_strs: Sequence[str]) -> Optional[openai.CompletionLogProbs]:
    """The same per-token records in the legacy completions layout: parallel lists of token strings, their
    log-probabilities, a ``{token: logprob}`` dict of alternatives and the offset of every token in the text."""
    if not json_strs:
        return None
    tokens, lps, tops, offsets = [], [], [], []
    at = 0
    for s in json_strs:
        d = json.loads(s)
        tokens.append(d["token"])
        lps.append(d["logprob"])
        tops.append({t["token"]: t["logprob"] for t in d.get("top_logprobs", [])})
        offsets.append(at)
        at += len(d["token"])
    return openai.CompletionLogProbs(text_offset=offsets, token_logprobs=lps, tokens=tokens, top_logprobs=tops)


def parse_usage(usage_json: Optional[str], include_extra: bool = True) -> Optional[openai.CompletionUsage]:
    if not usage_json:
        return None
    d = json.loads(usage_json)
    return openai.CompletionUsage(prompt_tokens=d.get("prompt_tokens", 0),
                                  completion_tokens=d.get("completion_tokens", 0),
                                  total_tokens=d.get("total_tokens", 0),
                                  extra=d.get("extra") if include_extra else None)


def convert_function_str_to_json(stringified_calls: str) -> List[Union[Dict, None]]:
    """``"[f(a=1), g(b='x')]"`` or a JSON tool-call object -> ``[{"name":..,"arguments":{..}}]``."""
    def visit(node):
        if isinstance(node, ast.Constant):
            return node.value
        if isinstance(node, ast.List):
            return [visit(e) for e in node.elts]
        if isinstance(node, ast.Dict):
            return {visit(k): visit(v) for k, v in zip(node.keys, node.values)}
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
            return -visit(node.operand)
        if isinstance(node, ast.Name):
            return node.id
        raise ValueError("unsupported expression in function call")

    text = stringified_calls.strip()
    try:
        obj = json.loads(text)
        calls = obj if isinstance(obj, list) else [obj]
        out = []
        for c in calls:
            if isinstance(c, dict) and "name" in c:
                out.append({"name": c["name"], "arguments": c.get("arguments", c.get("parameters", {}))})
        if out:
            return out
    except json.JSONDecodeError:
        pass
    try:
        tree = ast.parse(text, mode="eval").body
    except SyntaxError:
        return []
    nodes = tree.elts if isinstance(tree, (ast.List, ast.Tuple)) else [tree]
    result = []
    for n in nodes:
        if not isinstance(n, ast.Call):
            continue
        name = n.func.id if isinstance(n.func, ast.Name) else ast.unparse(n.func)
        try:
            args = {kw.arg: visit(kw.value) for kw in n.keywords}
        except ValueError:
            continue
        result.append({"name": name, "arguments": args})
    return result


def process_function_call_output(output_texts: List[str], finish_reasons: List[Optional[str]]
                                 ) -> Tuple[bool, List[List[openai.ChatToolCall]]]:
    """Parse generated text as tool calls; on success finish reasons become ``tool_calls``."""
    n = len(output_texts)
    tool_calls_list: List[List[openai.ChatToolCall]] = [[] for _ in range(n)]
    ok = True
    for i, text in enumerate(output_texts):
        try:
            fns = convert_function_str_to_json(text)
        except (SyntaxError, ValueError):
            fns = []
        if not fns:
            ok = False
            continue
        tool_calls_list[i] = [openai.ChatToolCall(type="function", function=openai.ChatFunctionCall(
            name=f["name"], arguments=f["arguments"])) for f in fns if f is not None]
        if finish_reasons[i] == "stop":
            finish_reasons[i] = "tool_calls"
    return ok, tool_calls_list


def metrics_to_prometheus_text(metrics: Dict[str, Any], prefix: str = "") -> str:
    """Flatten the engine metrics JSON into Prometheus exposition lines."""
    lines: List[str] = []

    def walk(d, pre):
        for k, v in d.items():
            if isinstance(v, dict):
                walk(v, pre)
            elif isinstance(v, (int, float)) and not isinstance(v, bool):
                lines.append(f"{pre}{k}\t{v}")
    walk(metrics, prefix)
    return "\n".join(lines) + ("\n" if lines else "")
