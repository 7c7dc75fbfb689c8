"""Builds the run-time ``ParamStore`` of a (tensor-parallel / pipeline shard of a) model, either
from a converted-weight directory or from a seeded random initialisation.

Sharding follows the reference's per-weight strategies (``model/llama/llama_model.py:109-202`` and
``support/tensor_parallel.py:36-97``): ``qkv_proj`` / ``gate_up_proj`` / ``up_proj`` are split over
output features per segment, ``o_proj`` / ``down_proj`` over input features, expert weights
``e1_e3`` over dim 1 (segments [I, I]) and ``e2`` over dim 2; embeddings, norms and ``lm_head`` are
replicated.  With expert parallelism whole experts are distributed instead.  Group-quantised
weights are sharded in their packed form (rows freely; columns in units of one quantisation group).
"""

from __future__ import annotations

import os
from typing import Callable, Dict, Iterator, Optional, Tuple

import torch

from .. import quantization as Q
from ..ops import LinearWeight
from .config import ModelConfig
from .transformer import ParamStore, column_sharded, param_specs, shard_rows


def _quantized(kind: str, name: str, quant: Q.Quantization) -> bool:
    if quant.kind == "no-quant":
        return False
    if kind in ("linear", "experts"):
        if name.startswith("lm_head") and not quant.quantize_final_fc:
            return False
        return True
    if kind == "embedding":
        return quant.quantize_embedding and quant.kind == "group-quant"
    return False


def _stage_of_layer(cfg: ModelConfig, layer: int) -> int:
    per = -(-cfg.num_hidden_layers // max(1, cfg.pipeline_parallel_stages))
    return layer // per


def layer_partition(cfg: ModelConfig) -> list:
    s = max(1, cfg.pipeline_parallel_stages)
    per = -(-cfg.num_hidden_layers // s)
    return [min(i * per, cfg.num_hidden_layers) for i in range(s)] + [cfg.num_hidden_layers]


def _wanted(name: str, cfg: ModelConfig, layers: range) -> bool:
    if name.startswith(("vision_tower.", "multi_modal_projector.", "model.vision_embed_tokens.")) or name.endswith(".q_calibration_scale"):
        return False  # read by the vision tower / kept as calibration metadata, not by the decoder
    if name.startswith("model.layers."):
        li = int(name.split(".")[2])
        return li in layers
    if name.startswith("model.embed") or name.startswith("lm_head"):
        return True  # every stage keeps embedding and head (reference: llama_model.py:265-280)
    if name.startswith("model.norm"):
        return layers.stop == cfg.num_hidden_layers
    return True


def _shard_dense(name: str, w: torch.Tensor, kind: str, cfg: ModelConfig, tp: int, rank: int,
                 ep: bool) -> torch.Tensor:
    """Shard a full-precision tensor for `rank`."""
    if tp == 1:
        return w
    base = name.rsplit(".", 1)[0]
    if kind == "experts":
        if ep:
            per = w.shape[0] // tp
            return w[rank * per:(rank + 1) * per].contiguous()
        if base.endswith("e1_e3"):
            half = w.shape[1] // 2
            per = half // tp
            return torch.cat([w[:, rank * per:(rank + 1) * per], w[:, half + rank * per: half + (rank + 1) * per]],
                             dim=1).contiguous()
        per = w.shape[2] // tp
        return w[:, :, rank * per:(rank + 1) * per].contiguous()
    if kind in ("linear", "bias"):
        segs = shard_rows(base, cfg, tp, rank, w.shape[0])
        if segs is not None:
            return torch.cat([w[a:b] for a, b in segs], dim=0).contiguous()
        if kind == "linear" and column_sharded(base):
            per = w.shape[1] // tp
            return w[:, rank * per:(rank + 1) * per].contiguous()
    return w


def _make_linear(name: str, w: torch.Tensor, bias: Optional[torch.Tensor], quant: Q.Quantization,
                 quantize: bool, device: torch.device) -> LinearWeight:
    n, k = w.shape[-2], w.shape[-1]
    if not quantize:
        return LinearWeight("dense", w.to(quant.torch_dtype), None, bias, None, n, k).to(device)
    if quant.kind == "group-quant":
        qw, qs = Q.group_quantize(w, quant)
        return LinearWeight("q4", qw, qs, bias, quant, n, k).to(device)
    if quant.kind == "fp8-block-scale":
        qw, sc = Q.fp8_block_quantize(w, quant.block_size, quant.weight_dtype)
        return LinearWeight("fp8_block", qw, sc, bias, quant, n, k).to(device)
    if quant.kind == "fp8-per-tensor":
        qw, sc = Q.fp8_per_tensor_quantize(w, quant.weight_dtype)
        return LinearWeight("fp8_tensor", qw, sc, bias, quant, n, k).to(device)
    raise ValueError(f"quantization kind {quant.kind} is not supported at run time")


def _store(store: ParamStore, name: str, kind: str, w: torch.Tensor, quant: Q.Quantization,
           device: torch.device, biases: Dict[str, torch.Tensor]) -> None:
    base = name.rsplit(".", 1)[0]
    if kind in ("linear", "embedding"):
        q = _quantized(kind, name, quant)
        if kind == "embedding" and not q:
            store.tensors[name] = w.to(quant.torch_dtype).to(device)
            return
        if kind == "embedding":
            # the lookup kernel reads the artifact nibble order; keep it (a tied lm_head re-lays it out)
            qw, qs = Q.group_quantize(w, quant)
            lw = LinearWeight("q4", qw.to(device), qs.to(device), None, quant, w.shape[0], w.shape[1], False)
        else:
            lw = _make_linear(name, w, None, quant, q, device)
        store.linears[base] = lw
    elif kind == "experts":
        q = _quantized(kind, name, quant)
        store.linears[base] = _make_linear(name, w, None, quant, q, device)
    elif kind == "bias":
        biases[base] = w.to(quant.torch_dtype).to(device)
    elif kind == "router":
        store.tensors[name] = w.to(quant.torch_dtype).to(device)
    elif kind == "f32":
        store.tensors[name] = w.float().to(device)
    else:
        store.tensors[name] = w.to(quant.torch_dtype).to(device)


def random_params(cfg: ModelConfig, quant: Q.Quantization, seed: int, device: torch.device,
                  tp: int = 1, rank: int = 0, layers: Optional[range] = None, std: float = 0.02,
                  gen_device: Optional[torch.device] = None) -> ParamStore:
    """Weights ~ N(0, std) (norm weights = 1 - offset, biases = 0), identical on every rank before
    sharding because each tensor has its own generator seeded by (seed, name)."""
    layers = layers if layers is not None else range(cfg.num_hidden_layers)
    # CPU and CUDA generators give different streams: MLCB_RANDOM_INIT_DEVICE=cpu makes a GPU run and a CPU
    # run of the same seed hold the same weights (numerics tests against a CPU oracle)
    forced = os.environ.get("MLCB_RANDOM_INIT_DEVICE")
    gen_device = torch.device(forced) if forced else (gen_device or device)
    store = ParamStore()
    biases: Dict[str, torch.Tensor] = {}
    ep = cfg.expert_parallel and tp > 1
    for idx, (name, (shape, kind)) in enumerate(param_specs(cfg).items()):
        if not _wanted(name, cfg, layers):
            continue
        if kind == "norm":
            w = torch.full(shape, 1.0 - cfg.norm_weight_offset)
        elif kind == "bias":
            w = torch.zeros(shape)
        elif "time_mix_" in name or (name.endswith("time_decay") and len(shape) == 2) or \
                ("time_maa_" in name and len(shape) == 1):
            # interpolation weights and decays of recurrent blocks live in (0, 1)
            g = torch.Generator(device=gen_device)
            g.manual_seed((seed * 1000003 + idx * 7919) % (2 ** 63 - 1))
            w = torch.rand(shape, generator=g, device=gen_device, dtype=torch.float32) * 0.7 + 0.25
        else:
            g = torch.Generator(device=gen_device)
            g.manual_seed((seed * 1000003 + idx * 7919) % (2 ** 63 - 1))
            w = torch.randn(shape, generator=g, device=gen_device, dtype=torch.float32) * std
            w = w.to(quant.torch_dtype if quant.torch_dtype != torch.float32 else torch.float32)
        w = _shard_dense(name, w, kind, cfg, tp, rank, ep)
        _store(store, name, kind, w, quant, device, biases)
        del w
    for base, b in biases.items():
        if base in store.linears:
            store.linears[base].bias = b
        else:
            store.tensors[base + ".bias"] = b
    return store


def _shard_packed(name_base: str, qw: torch.Tensor, qs: torch.Tensor, cfg: ModelConfig, quant: Q.Quantization,
                  tp: int, rank: int, ep: bool, experts: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Shard a group-quantised weight without unpacking."""
    if tp == 1:
        return qw, qs
    wpg = quant.words_per_group
    if experts:
        if ep:
            per = qw.shape[0] // tp
            return qw[rank * per:(rank + 1) * per].contiguous(), qs[rank * per:(rank + 1) * per].contiguous()
        if name_base.endswith("e1_e3"):
            half = qw.shape[1] // 2
            per = half // tp
            sel = lambda t: torch.cat([t[:, rank * per:(rank + 1) * per],
                                       t[:, half + rank * per: half + (rank + 1) * per]], dim=1).contiguous()
            return sel(qw), sel(qs)
        groups = qs.shape[2] // tp
        return (qw[:, :, rank * groups * wpg:(rank + 1) * groups * wpg].contiguous(),
                qs[:, :, rank * groups:(rank + 1) * groups].contiguous())
    segs = shard_rows(name_base, cfg, tp, rank, qw.shape[0])
    if segs is not None:
        return (torch.cat([qw[a:b] for a, b in segs], 0).contiguous(),
                torch.cat([qs[a:b] for a, b in segs], 0).contiguous())
    if column_sharded(name_base):
        groups = qs.shape[1] // tp
        return (qw[:, rank * groups * wpg:(rank + 1) * groups * wpg].contiguous(),
                qs[:, rank * groups:(rank + 1) * groups].contiguous())
    return qw, qs


def load_params(model_dir: str, cfg: ModelConfig, quant: Q.Quantization, device: torch.device,
                tp: int = 1, rank: int = 0, layers: Optional[range] = None,
                progress: Optional[Callable[[str], None]] = None) -> ParamStore:
    """Load ``tensor-cache.json`` + shards, shard for `rank`, and move to `device`.
    Pre-sharded checkpoints (``{name}_shard-{rank}`` entries) are read directly."""
    from ..loader.tensor_cache import TensorCache  # pylint: disable=import-outside-toplevel

    cache = TensorCache(model_dir)
    layers = layers if layers is not None else range(cfg.num_hidden_layers)
    specs = param_specs(cfg)
    store = ParamStore()
    biases: Dict[str, torch.Tensor] = {}
    ep = cfg.expert_parallel and tp > 1
    pend_q: Dict[str, Dict[str, torch.Tensor]] = {}
    presharded = any(n.endswith(f"_shard-{rank}") for n in cache.names())
    suffix = f"_shard-{rank}"
    for raw_name, t in cache:
        name = raw_name
        this_presharded = False
        if "_shard-" in raw_name:
            if not raw_name.endswith(suffix):
                continue
            name = raw_name[: -len(suffix)]
            this_presharded = True
        if not _wanted(name, cfg, layers):
            continue
        if progress:
            progress(name)
        base, leaf = name.rsplit(".", 1)
        if leaf in ("q_weight", "q_scale"):
            slot = pend_q.setdefault(base, {})
            slot[leaf] = t
            if len(slot) == 2:
                spec_name = base + ".weight"
                kind = specs.get(spec_name, (None, "linear"))[1]
                qw, qs = slot["q_weight"], slot["q_scale"]
                if not this_presharded:
                    qw, qs = _shard_packed(base, qw, qs, cfg, quant, tp, rank, ep, kind == "experts")
                n = qw.shape[-2]
                k = qs.shape[-1] * quant.group_size
                lw = LinearWeight("q4", qw, qs.to(quant.torch_dtype), None, quant, n, k)
                store.linears[base] = lw if kind == "embedding" else lw.to(device)
                if kind == "embedding":
                    store.linears[base] = LinearWeight("q4", qw.to(device), qs.to(quant.torch_dtype).to(device),
                                                       None, quant, n, k, False)
                del pend_q[base]
            continue
        if leaf == "weight_scale_inv":
            pend_q.setdefault(base, {})["scale"] = t
            continue
        kind = specs.get(name, (None, "norm"))[1]
        if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and leaf == "weight":
            slot = pend_q.setdefault(base, {})
            slot["w"] = t
            continue
        if not this_presharded:
            t = _shard_dense(name, t, kind, cfg, tp, rank, ep)
        if kind in ("linear", "experts"):
            store.linears[base] = LinearWeight("dense", t.to(quant.torch_dtype), None, None, None,
                                               t.shape[-2], t.shape[-1]).to(device)
        elif kind == "bias":
            biases[base] = t.to(quant.torch_dtype).to(device)
        elif kind == "f32":
            store.tensors[name] = t.float().to(device)
        else:
            store.tensors[name] = t.to(quant.torch_dtype).to(device)
    # fp8 block-scale pairs
    for base, slot in pend_q.items():
        if "w" in slot and "scale" in slot:
            w, sc = slot["w"], slot["scale"]
            store.linears[base] = LinearWeight("fp8_block", w.to(device), sc.float().to(device), None, quant,
                                               w.shape[-2], w.shape[-1])
    for base, b in biases.items():
        if base in store.linears:
            store.linears[base].bias = b
        else:
            store.tensors[base + ".bias"] = b
    return store


def export_params(cfg: ModelConfig, quant: Q.Quantization, named_full: Iterator[Tuple[str, torch.Tensor]]
                  ) -> Iterator[Tuple[str, torch.Tensor]]:
    """Turn full-precision MLC-named tensors into the on-disk parameter set of `quant`
    (``*.q_weight`` / ``*.q_scale`` for group quantisation, fp8 + scales for the fp8 modes)."""
    specs = param_specs(cfg)
    for name, w in named_full:
        kind = specs.get(name, (None, "norm"))[1]
        base = name.rsplit(".", 1)[0]
        if _quantized(kind, name, quant):
            if quant.kind == "group-quant":
                qw, qs = Q.group_quantize(w, quant)
                yield base + ".q_weight", qw
                yield base + ".q_scale", qs
                continue
            if quant.kind == "fp8-block-scale" and kind != "embedding":
                qw, sc = Q.fp8_block_quantize(w, quant.block_size, quant.weight_dtype)
                yield base + ".weight", qw
                yield base + ".weight_scale_inv", sc
                continue
            if quant.kind == "fp8-per-tensor" and kind != "embedding":
                qw, sc = Q.fp8_per_tensor_quantize(w, quant.weight_dtype)
                yield base + ".q_weight", qw
                yield base + ".q_scale", sc
                continue
        yield name, w.to(quant.torch_dtype)


def load_hf_params(hf_dir: str, cfg: ModelConfig, quant: Q.Quantization, device: torch.device,
                   tp: int = 1, rank: int = 0, layers: Optional[range] = None) -> ParamStore:
    """Build the run-time parameters straight from a HuggingFace checkpoint, quantising on the fly
    (the in-memory form of ``convert_weight`` followed by ``load_params``)."""
    from ..loader.huggingface_loader import iter_mlc_params  # pylint: disable=import-outside-toplevel

    layers = layers if layers is not None else range(cfg.num_hidden_layers)
    specs = param_specs(cfg)
    store = ParamStore()
    biases: Dict[str, torch.Tensor] = {}
    ep = cfg.expert_parallel and tp > 1
    for name, w in iter_mlc_params(hf_dir, cfg):
        if not _wanted(name, cfg, layers):
            continue
        kind = specs[name][1]
        w = _shard_dense(name, w.to(device if device.type == "cuda" else "cpu"), kind, cfg, tp, rank, ep)
        _store(store, name, kind, w, quant, device, biases)
    for base, b in biases.items():
        if base in store.linears:
            store.linears[base].bias = b
        else:
            store.tensors[base + ".bias"] = b
    return store
