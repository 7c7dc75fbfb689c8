"""Model executor: the Python side of the native engine's ``ModelBackend``.

One call per scheduling step: the engine hands over the KV manager's index arrays and the sampling
parameters as NumPy arrays; the executor packs them into one pinned staging buffer, uploads it with
a single asynchronous copy (and, under tensor parallelism, one broadcast to the other ranks), runs
the model, processes logits and samples on the device, and reads back only the sampled tokens.

Reference counterparts: ``cpp/serve/model.cc:245-367,455-534,682-768`` (batch prefill / decode /
verify wrappers), ``cpp/serve/logit_processor.cc:40-458`` and ``cpp/serve/sampler/gpu_sampler.cc``
(host-side packing for the logit-processing and sampling kernels).
"""

from __future__ import annotations

import collections
import ctypes
import json
import os
import time

from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..models.transformer import BatchInfo, DecoderModel

_INT_KEYS = ("positions", "slots", "q_seq", "q_kvlen", "q_kvstart", "page_indptr", "page_indices",
             "page_copies", "q_indptr", "seq_lens", "append_lens")
_S_INT = ("logit_token_index", "top_k", "pen_row", "pen_token", "pen_count", "bias_row", "bias_token",
          "mask_rows", "mask_bits", "prob_slots")
_S_FLT = ("temperature", "top_p", "uniform", "penalties", "bias_value")


# KV pools exported by engines of this process (disaggregated serving inside one process)
_LOCAL_KV_POOLS: Dict[str, torch.Tensor] = {}
_KV_DTYPES = {"torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32,
              "torch.float8_e4m3fn": torch.float8_e4m3fn}


def _pad4(n: int) -> int:
    return (n + 3) & ~3


def graph_bucket(n: int) -> int:
    """Batch size a decode step of ``n`` sequences is padded to before it is run from a CUDA graph: the next
    power of two up to 32, then the next multiple of 16. A serving trace whose batch drifts by a few
    sequences per step then replays a handful of graphs instead of capturing one per batch size."""
    if n <= 32:
        b = 1
        while b < n:
            b *= 2
        return b
    return (n + 15) // 16 * 16


def pad_decode_arrays(arrays: Dict[str, np.ndarray], target: int) -> None:
    """Append ``target - n`` stand-in sequences to the packed arrays of a pure decode step (in place).

    A stand-in feeds token 0 at position 0, appends nothing to the cache (slot -1) and attends to the first
    token of page 0, so its row stays finite and nothing it computes is read: the sampling rows index
    the real sequences only."""
    n = int(arrays["q_indptr"].size) - 1
    extra = target - n
    if extra <= 0:
        return
    i32 = np.int32

    def cat(key, tail):
        arrays[key] = np.concatenate([arrays[key], np.asarray(tail, dtype=i32)])

    cat("token_ids", np.zeros(extra))
    cat("positions", np.zeros(extra))
    cat("slots", np.full(extra, -1))
    cat("q_seq", np.arange(n, target))
    cat("q_kvlen", np.ones(extra))
    last = int(arrays["page_indptr"][-1])
    cat("page_indptr", last + 1 + np.arange(extra))
    cat("page_indices", np.zeros(extra))
    cat("q_indptr", n + 1 + np.arange(extra))
    cat("seq_lens", np.ones(extra))
    cat("append_lens", np.ones(extra))
    if "token_src" in arrays:
        cat("token_src", np.full(extra, -1))


def split_plan(plan: dict, token_ids: np.ndarray, sp: dict, s: int):
    """Cut one forward plan at sequence ``s`` into two that can run one after the other: sequences
    ``[0, s)`` and ``[s, n)`` with their tokens, pages and logit rows (indices rebased). The first part
    carries only its logit rows; the second carries the sampling parameters of all rows, since the rows of
    both parts are sampled together once the second part's logits exist. Copy-on-write page copies run with
    the first part."""
    qi = np.asarray(plan["q_indptr"], dtype=np.int64)
    pi = np.asarray(plan["page_indptr"], dtype=np.int64)
    n = qi.size - 1
    if not 0 < s < n:
        raise ValueError(f"cannot split {n} sequences at {s}")
    t, pg = int(qi[s]), int(pi[s])
    tok_keys = ("positions", "slots", "q_seq", "q_kvlen", "q_kvstart", "tree_mask")
    seq_keys = ("seq_lens", "append_lens", "seq_ids")
    parts = []
    for lo_s, hi_s, lo_t, hi_t, lo_p, hi_p in ((0, s, 0, t, 0, pg), (s, n, t, int(qi[-1]), pg, int(pi[-1]))):
        p = {}
        for k in tok_keys:
            a = np.asarray(plan[k])
            p[k] = a[lo_t:hi_t] if a.size else a
        p["q_seq"] = np.asarray(p["q_seq"]) - lo_s
        for k in seq_keys:
            if k in plan:
                p[k] = np.asarray(plan[k])[lo_s:hi_s]
        p["q_indptr"] = qi[lo_s:hi_s + 1] - lo_t
        p["page_indptr"] = pi[lo_s:hi_s + 1] - lo_p
        p["page_indices"] = np.asarray(plan["page_indices"])[lo_p:hi_p]
        p["page_copies"] = np.asarray(plan["page_copies"]) if lo_s == 0 else np.zeros(0, np.int32)
        p["max_seq_len"] = int(np.max(p["seq_lens"])) if len(p["seq_lens"]) else 0
        parts.append(p)
    rows = np.asarray(sp["logit_token_index"], dtype=np.int64)
    first = rows < t
    if first.any() and not first[: int(first.sum())].all():
        raise ValueError("logit rows are not ordered by sequence")
    sp_a = {k: (np.zeros(0, np.float32) if k in _S_FLT else np.zeros(0, np.int32)) for k in _S_INT + _S_FLT}
    for k, v in sp.items():
        if k not in sp_a:
            sp_a[k] = v[:0] if isinstance(v, (np.ndarray, list)) else v
    sp_a["logit_token_index"] = rows[first]
    sp_b = dict(sp)
    sp_b["logit_token_index"] = rows[~first] - t
    tok = np.asarray(token_ids)
    return [(parts[0], tok[:t], sp_a), (parts[1], tok[t:], sp_b)]


class FeatureStore:
    """Target-model features (final-normed hidden states) of the positions that a speculative draft
    head (EAGLE, Medusa) has not consumed yet, per sequence, plus the head's own latest prediction.

    The draft head reads the feature of position ``p - 1`` together with the token at position ``p``
    (reference: ``cpp/serve/engine_actions/eagle_new_request_prefill.cc`` and ``eagle_batch_draft.cc``
    move the same rows through the draft-token workspace).  While the target has computed that position
    the true feature is used; beyond it, the head continues from its own previous output.
    """

    CAP_ROWS = 512    # per sequence: older rows are dropped (the head then sees zeros for them)
    CAP_SEQS = 4096   # sequences remembered; the least recently written go first

    def __init__(self):
        self.rows: "collections.OrderedDict[int, tuple]" = collections.OrderedDict()
        self.pred: Dict[int, tuple] = {}
        # draft trees: the head's outputs for every node of the tree it was last fed (row j = node j); a node
        # of the next, larger tree continues from its parent's row
        self.tree: Dict[int, torch.Tensor] = {}

    def put(self, seq: int, start: int, feats: torch.Tensor) -> None:
        """Rows for positions ``start ..``; anything stored from ``start`` on is replaced."""
        feats = feats.detach().clone()
        cur = self.rows.pop(seq, None)
        if cur is not None:
            s0, t = cur
            if s0 <= start <= s0 + t.shape[0]:
                feats = torch.cat([t[: start - s0], feats])
                start = s0
        if feats.shape[0] > self.CAP_ROWS:
            start += feats.shape[0] - self.CAP_ROWS
            feats = feats[-self.CAP_ROWS:]
        self.rows[seq] = (start, feats)
        self.pred.pop(seq, None)
        self.tree.pop(seq, None)
        while len(self.rows) > self.CAP_SEQS:
            old, _ = self.rows.popitem(last=False)
            self.pred.pop(old, None)
            self.tree.pop(old, None)

    def end(self, seq: int) -> int:
        """One past the last position whose true feature is known (0: none)."""
        cur = self.rows.get(seq)
        return 0 if cur is None else cur[0] + cur[1].shape[0]

    def span(self, seq: int):
        cur = self.rows.get(seq)
        return (0, None) if cur is None else cur

    def trim(self, seq: int, keep_from: int) -> None:
        cur = self.rows.get(seq)
        if cur is not None and keep_from > cur[0]:
            s0, t = cur
            k = min(keep_from - s0, t.shape[0] - 1)  # always keep the newest row
            if k > 0:
                self.rows[seq] = (s0 + k, t[k:])

    def fork(self, parent: int, child: int) -> None:
        """Parallel samples: the child continues from what is known about its parent (rows are never edited in
        place, so sharing the tensors is safe)."""
        cur = self.rows.get(parent)
        if cur is not None:
            self.rows[child] = cur
        if parent in self.pred:
            self.pred[child] = self.pred[parent]

    def clear(self) -> None:
        self.rows.clear()
        self.pred.clear()
        self.tree.clear()


class StagingBuffer:
    """Packs many small int32 / float32 arrays into one pinned buffer -> one H2D copy."""

    def __init__(self, device: torch.device, capacity: int = 1 << 16):
        self.device = device
        self.capacity = 0
        self.host = None
        self.dev = None
        self._grow(capacity)

    def _grow(self, n: int) -> None:
        cap = max(n, self.capacity * 2, 1 << 12)
        self.generation = getattr(self, "generation", 0) + 1  # device addresses change: drop CUDA graphs
        pin = self.device.type == "cuda"
        # two pinned host buffers used in turn: with deferred-read decode steps the host packs step n + 1
        # while the copy of step n may still be queued behind step n - 1's kernels
        self.hosts = [torch.empty(cap, dtype=torch.int32, pin_memory=pin) for _ in range(2 if pin else 1)]
        self.hosts_np = [h.numpy() for h in self.hosts]
        self.turn = 0
        self.host, self.host_np = self.hosts[0], self.hosts_np[0]
        self.dev = torch.empty(cap, dtype=torch.int32, device=self.device) if pin else self.host
        self.capacity = cap

    def upload(self, arrays: Dict[str, np.ndarray]) -> Dict[str, torch.Tensor]:
        total = sum(_pad4(a.size * (2 if a.dtype.itemsize == 8 else 1)) for a in arrays.values())
        if total > self.capacity:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)  # queued copies still read the old buffers
            self._grow(total)
        self.turn = (self.turn + 1) % len(self.hosts)
        self.host, self.host_np = self.hosts[self.turn], self.hosts_np[self.turn]
        off = 0
        layout = []
        # Fixed-size forward arrays first, the page list (the one array that grows from step to step
        # at a constant batch) next, sampling arrays last: the device address of every array a
        # captured forward reads then depends on the batch shape only.
        order = [k for k in arrays if not k.startswith("s_") and k != "page_indices"]
        order += [k for k in arrays if k == "page_indices"] + [k for k in arrays if k.startswith("s_")]
        for name in order:
            a = arrays[name]
            words = a.size * (2 if a.dtype.itemsize == 8 else 1)
            if words:
                self.host_np[off:off + words] = a.reshape(-1).view(np.int32)
            layout.append((name, off, words, a.dtype))
            off += _pad4(words)
        if self.dev is not self.host and off:
            self.dev[:off].copy_(self.host[:off], non_blocking=True)
        self.last_words = off
        return self.views(layout)

    def views(self, layout) -> Dict[str, torch.Tensor]:
        out = {}
        for name, off, words, dt in layout:
            t = self.dev[off:off + words]
            if dt == np.float32:
                t = t.view(torch.float32)
            elif dt.itemsize == 8:
                t = t.view(torch.int64)
            out[name] = t
        return out


class ModelExecutor:
    """Runs one or more ``DecoderModel`` (main model, optional draft model) for the engine."""

    def __init__(self, models: List[DecoderModel], device: torch.device, comm=None,
                 max_draft_slots: int = 0):
        self.models = models
        self.device = device
        self.comm = comm
        self.staging = StagingBuffer(device)
        self.vocab = models[0].cfg.vocab_size
        self.draft_probs: Optional[torch.Tensor] = None
        self.max_draft_slots = max_draft_slots
        self.embeddings: Dict[int, torch.Tensor] = {}
        self._next_embed = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launch_estimate = 0
        self.use_tensor_core_attention = device.type == "cuda"
        # CUDA graphs of decode-shaped forwards, keyed by the batch shape (MLCB_CUDA_GRAPH=0 disables).
        # Multi-rank engines capture only the fused tensor-parallel forward, whose collectives are this
        # library's kernels over peer memory (see _graph_ok): a forward with NCCL collectives inside did
        # not complete under capture in a two-rank run and stays on eager launches.
        self.use_graphs = device.type == "cuda" and os.environ.get("MLCB_CUDA_GRAPH", "1") != "0"
        self._graphs: Dict[tuple, dict] = {}
        self.graph_buckets = os.environ.get("MLCB_GRAPH_BUCKETS", "1") != "0"
        self._graph_pool = None
        self.graph_replays = 0
        self.graph_eligible_steps = 0  # steps that could run from a graph (replayed, captured or first seen)
        # pipeline stages: steps with at least this many tokens run as two micro-batches (0 = never)
        self.pp_microbatch_min_tokens = int(os.environ.get("MLCB_PP_MICROBATCH_MIN_TOKENS", "512"))
        self.pp_microbatch_steps = 0
        self._part_logits: List[torch.Tensor] = []
        self._nvtx = device.type == "cuda" and os.environ.get("MLCB_NVTX", "0") == "1"
        # speculative draft heads fed with the target's features: model id -> "eagle" | "medusa"
        self.spec_heads: Dict[int, str] = {}
        for mi, m in enumerate(models):
            if mi > 0 and m.cfg.extra.get("eagle"):
                self.spec_heads[mi] = "eagle"
            elif mi > 0 and m.cfg.extra.get("medusa"):
                self.spec_heads[mi] = "medusa"
        # Tensor-parallel engines: a Medusa head is a few small matrices and no state, so rank 0 evaluates it
        # alone (every rank holds a copy); an EAGLE head is a sharded decoder layer that all ranks run, and rank
        # 0, which alone keeps the feature store, sends them the feature rows of each call.
        if self.spec_heads and comm is not None and comm.pp_size > 1:
            raise NotImplementedError("EAGLE / Medusa draft heads are not available with pipeline stages")
        self.features = FeatureStore()
        # wall-clock seconds the host spent per phase of forward_sample (profiling aid)
        self.host_times: Dict[str, float] = {"pack": 0.0, "broadcast": 0.0, "upload": 0.0, "forward": 0.0,
                                             "logits_sample": 0.0, "readback": 0.0, "calls": 0.0}
        self.graph_launches = 0
        # deferred-read decode steps: tokens of the last launched step (device), results not read yet
        self._last_tokens: Dict[int, torch.Tensor] = {}
        self._pending: "collections.deque[dict]" = collections.deque()
        self._readback_turn = 0
        self._readback_bufs: List[Dict[str, torch.Tensor]] = [{}, {}]

    # ------------------------------------------------------------------ embeddings (multimodal)
    def _enter(self) -> None:
        """Kernels launch on the calling thread's current CUDA device; the engine drives this object
        from its own threads, whose current device starts at 0."""
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)

    def hold_embedding(self, emb: torch.Tensor) -> int:
        h = self._next_embed
        self._next_embed += 1
        self.embeddings[h] = emb.to(self.device)
        return h

    def release_embedding(self, handle: int) -> None:
        self.embeddings.pop(int(handle), None)

    def reset(self) -> None:
        self.embeddings.clear()
        self.features.clear()
        self._pending.clear()
        self._last_tokens.clear()

    def synchronize(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ plumbing
    def _batch_info(self, dev: Dict[str, torch.Tensor], plan: dict, model: DecoderModel) -> BatchInfo:
        b = BatchInfo(
            positions=dev["positions"], slots=dev["slots"], q_seq=dev["q_seq"], q_kvlen=dev["q_kvlen"],
            page_indptr=dev["page_indptr"], page_indices=dev["page_indices"],
            q_kvstart=dev["q_kvstart"] if dev["q_kvstart"].numel() else None,
            tree_mask=dev["tree_mask"] if dev["tree_mask"].numel() else None,
            num_tokens=int(dev["positions"].numel()))
        if getattr(model, "stateful", False):
            # recurrent models select their state by sequence id and need the chunk boundaries on the host
            qi = np.asarray(plan["q_indptr"])
            pos = np.asarray(plan["positions"])
            b.seq_ids = np.asarray(plan["seq_ids"])
            b.seq_forks = np.asarray(plan.get("seq_forks", ()), dtype=np.int64).reshape(-1, 2)
            b.q_indptr = qi
            b.start_positions = np.asarray([int(pos[qi[i]]) if qi[i + 1] > qi[i] else 0
                                            for i in range(len(qi) - 1)])
        if "tile_seq" in dev and self._tc_attention_ok(model):
            from ..ops.attention import AttentionPlan  # pylint: disable=import-outside-toplevel

            from ..ops.attention import choose_splits  # pylint: disable=import-outside-toplevel

            n_dec = int(dev["dec_seq"].numel())
            max_pages = (int(plan["max_seq_len"]) + 15) // 16
            b.attn_plan = AttentionPlan(dev["tile_seq"], dev["tile_qstart"], dev["tile_ntok"], b.q_kvlen,
                                        b.page_indptr, b.page_indices, int(dev["tile_seq"].numel()),
                                        dec_seq=dev["dec_seq"], dec_qstart=dev["dec_qstart"],
                                        dec_ntok=dev["dec_ntok"], num_dec=n_dec,
                                        dec_splits=choose_splits(n_dec, model.hkv, max_pages, self.device)
                                        if n_dec else 1, max_pages=max_pages)
        return b

    def _tc_attention_ok(self, model: DecoderModel) -> bool:
        return (self.use_tensor_core_attention and model.d == 128 and model.page == 16
                and model.kv_dtype in (torch.float16, torch.bfloat16))

    @staticmethod
    def _masked_attention(model: DecoderModel) -> bool:
        """Models some of whose layers always need the masked attention variant (windows or chunks per
        layer, logit soft-capping)."""
        return model.cfg.layer_attn_kinds is not None or model.cfg.attn_logit_softcap != 0

    def _pack(self, plan: dict, token_ids: np.ndarray, sp: Optional[dict], model_id: int = 0
              ) -> Dict[str, np.ndarray]:
        arrays: Dict[str, np.ndarray] = {"token_ids": np.ascontiguousarray(token_ids, dtype=np.int32)}
        for k in _INT_KEYS:
            arrays[k] = np.ascontiguousarray(plan[k], dtype=np.int32)
        arrays["tree_mask"] = np.ascontiguousarray(plan["tree_mask"], dtype=np.uint64).view(np.int64)
        model = self.models[model_id]
        if getattr(model, "stateful", False):
            # recurrent models pick their state by sequence id: the other ranks need the ids too
            arrays["seq_ids"] = np.ascontiguousarray(plan["seq_ids"], dtype=np.int32)
            arrays["seq_forks"] = np.ascontiguousarray(plan.get("seq_forks", ()), dtype=np.int32)
        if self._pads_decode(model_id, arrays):
            pad_decode_arrays(arrays, graph_bucket(int(arrays["q_indptr"].size) - 1))
        if self._tc_attention_ok(model):
            from ..ops.attention import build_tiles  # pylint: disable=import-outside-toplevel

            arrays.update(build_tiles(arrays["q_indptr"], model.hq // model.hkv))
        if sp is not None:
            for k in _S_INT:
                arrays["s_" + k] = np.ascontiguousarray(sp[k], dtype=np.int32)
            for k in _S_FLT:
                arrays["s_" + k] = np.ascontiguousarray(sp[k], dtype=np.float32)
        return arrays

    def _graph_candidate(self, model_id: int) -> bool:
        """What a model must be for any of its steps to run from a CUDA graph (see ``_graph_ok``)."""
        model = self.models[model_id]
        multi = self.comm is not None and self.comm.world_size > 1
        if multi and getattr(model, "fused", None) is None:
            return False
        # (an expert-parallel model qualifies through the fused forward: its exchanges are this package's
        # kernels with call numbers in device memory; its NCCL forward is not captured)
        ep_ok = getattr(model, "ep", None) is None or (
            getattr(model, "fused", None) is not None
            # the exchange buffers alternate between two parities: a replayed forward must start on the parity
            # it was captured with, so it has to contain an even number of exchanges
            and sum(1 for li in model.layers if model.cfg.is_moe_layer(li)) % 2 == 0)
        return (self.use_graphs and not self._pipeline(model_id) and ep_ok
                and not getattr(model, "stateful", False) and self._tc_attention_ok(model)
                and not self._masked_attention(model))

    def _pads_decode(self, model_id: int, arrays: Dict[str, np.ndarray]) -> bool:
        """Pure decode steps (one appended token per sequence, no tree, window or copy-on-write) of a model
        that runs from graphs are padded to a bucket size (``MLCB_GRAPH_BUCKETS=0`` keeps exact shapes)."""
        if not self.graph_buckets or not self._graph_candidate(model_id):
            return False
        qi = arrays["q_indptr"]
        n = int(qi.size) - 1
        model = self.models[model_id]
        return (n > 0 and int(qi[-1]) == n and arrays["token_ids"].size == n
                and arrays["tree_mask"].size == 0 and arrays["q_kvstart"].size == 0
                and arrays["page_copies"].size == 0 and (model.hq // model.hkv) <= 16)

    def _run_model(self, model_id: int, plan: dict, dev: Dict[str, torch.Tensor],
                   embed_handles: Optional[np.ndarray]) -> torch.Tensor:
        model = self.models[model_id]
        if dev["page_copies"].numel():
            model.copy_pages(dev["page_copies"])
        if self._graph_ok(model_id, dev, embed_handles):
            self.graph_eligible_steps += 1
            return self._run_graph(model_id, plan, dev)
        return self._run_eager(model_id, plan, dev, embed_handles)

    # ------------------------------------------------------------------ CUDA graphs
    def _graph_ok(self, model_id: int, dev: Dict[str, torch.Tensor], embed_handles) -> bool:
        """Pure decode-shaped steps (every sequence appends a few tokens through the decode attention
        kernel, no tree, no window, no copy-on-write) of a single-stage model: everything the forward
        launches then depends on the batch shape only.  Across ranks only the fused tensor-parallel
        forward is captured: its collectives are this library's kernels over peer memory (call numbers
        come from device memory), so the graph holds no NCCL call."""
        return (self._graph_candidate(model_id) and embed_handles is None
                and "dec_seq" in dev and dev["dec_seq"].numel() > 0 and dev["tile_seq"].numel() == 0
                and dev["page_copies"].numel() == 0 and dev["tree_mask"].numel() == 0
                and dev["q_kvstart"].numel() == 0)

    def _run_graph(self, model_id: int, plan: dict, dev: Dict[str, torch.Tensor]) -> torch.Tensor:
        from ..ops.attention import choose_splits  # pylint: disable=import-outside-toplevel

        model = self.models[model_id]
        max_pages = (int(plan["max_seq_len"]) + 15) // 16
        splits = choose_splits(int(dev["dec_seq"].numel()), model.hkv, max_pages, self.device)
        shape = tuple((k, int(v.numel())) for k, v in dev.items() if not k.startswith("s_") and k != "page_indices")
        key = (model_id, self.staging.generation, splits, shape)
        entry = self._graphs.get(key)
        if entry is None:
            # first sight of a shape: run it eagerly (lazy one-time set-up must not happen under capture;
            # every rank takes the same decision from the same broadcast arrays)
            if len(self._graphs) >= 64:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = {"graph": None}
            return self._run_eager(model_id, plan, dev, None)
        if entry["graph"] is None:
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            from ..ops._lib import lib  # pylint: disable=import-outside-toplevel

            lib().mlcb_launch_count.restype = ctypes.c_longlong
            before = lib().mlcb_launch_count()
            fused = getattr(model, "fused", None)
            base = fused.base if fused is not None else 0
            ep = getattr(model, "ep", None)
            ep_base = ep.base if ep is not None else 0
            multi = self.comm is not None and self.comm.world_size > 1
            with torch.cuda.graph(graph, pool=self._graph_pool,
                                  capture_error_mode="thread_local" if multi else "global"):
                hidden = self._run_eager(model_id, plan, dev, None)
                normed = getattr(model, "_final_normed", None)
            calls = 0
            if fused is not None:
                # nothing ran during capture: the call-number base moves when the graph is replayed
                calls, fused.base = fused.base - base, base
                if calls % 2:
                    raise RuntimeError("a captured fused forward must make an even number of reduce-scatter calls")
            ep_calls = 0
            if ep is not None:
                # the same for the expert exchanges; buffer parities repeat only after an even number of them
                ep_calls, ep.base = ep.base - ep_base, ep_base
                if ep_calls % 2:
                    raise RuntimeError("a captured forward must make an even number of expert exchanges")
            entry.update(graph=graph, hidden=hidden, normed=normed, fused_calls=calls, ep_calls=ep_calls,
                         launches=int(lib().mlcb_launch_count() - before))
        entry["graph"].replay()
        if entry.get("fused_calls"):
            model.fused.note_replay(entry["fused_calls"])
        if entry.get("ep_calls"):
            model.ep.note_replay(entry["ep_calls"])
        self.graph_replays += 1
        self.graph_launches += entry["launches"]  # kernels a replay launches (the C counter sees captures only)
        model._final_normed = entry["normed"]  # pylint: disable=protected-access
        return entry["hidden"]

    def _run_eager(self, model_id: int, plan: dict, dev: Dict[str, torch.Tensor],
                   embed_handles: Optional[np.ndarray]) -> torch.Tensor:
        model = self.models[model_id]
        b = self._batch_info(dev, plan, model)
        staged = self._pipeline(model_id)
        if staged and not model.first_stage:
            # hidden state of the previous pipeline stage (same tensor-parallel rank)
            x = torch.empty(b.num_tokens, model.cfg.hidden_size, dtype=model.dtype, device=self.device)
            self.comm.recv_from_prev_stage(x)
        else:
            x = model.embed(dev["token_ids"])
            if embed_handles is not None:
                # rows of held embeddings (images) replace the table lookups: one gather per image, indexed
                # on the device by the row numbers the engine put in place of token ids
                idx = np.nonzero(embed_handles >= 0)[0]
                for h in np.unique(embed_handles[idx]):
                    sel = torch.from_numpy(idx[embed_handles[idx] == h]).to(self.device)
                    rows = dev["token_ids"][sel].long()
                    x[sel] = self.embeddings[int(h)].to(x.dtype)[rows]
        h = model.forward(x, b)
        if staged and not model.last_stage:
            self.comm.send_to_next_stage(h)
        return h

    def _pipeline(self, model_id: int) -> bool:
        return self.comm is not None and self.comm.pp_size > 1 and model_id == 0

    def _pipeline_parts(self, model_id: int, plan: dict, token_ids: np.ndarray, embed_handles, sp: dict):
        """Prefill-sized steps of a pipelined model run as two micro-batches: while a later stage works on
        the first half of the sequences, the stage before it already computes the second half (the hand-over
        is a stream-ordered NCCL send, so nothing waits on the host). Every stage reads its weights once per
        part, so steps with few tokens, which are bound by those reads, stay whole. The last stage keeps the
        first part's logits and returns the rows of both parts in one message.
        Returns ``None`` (run whole) or ``(device arrays of the last part, hidden of the last part)``."""
        if not self._pipeline(model_id) or embed_handles is not None or self.spec_heads \
                or self.pp_microbatch_min_tokens <= 0:
            return None
        qi = np.asarray(plan["q_indptr"], dtype=np.int64)
        n, total = qi.size - 1, int(qi[-1]) if qi.size else 0
        if n < 2 or total < self.pp_microbatch_min_tokens:
            return None
        s = int(np.searchsorted(qi, total / 2.0))
        s = min(max(s, 1), n - 1)
        parts = split_plan(plan, token_ids, sp, s)
        dev = hidden = None
        for i, (p, tok, spx) in enumerate(parts):
            arrays = self._pack(p, tok, spx, model_id)
            self.comm.broadcast_step("forward" if i == len(parts) - 1 else "forward_part", model_id,
                                     {k: v for k, v in arrays.items()
                                      if not k.startswith("s_") or k == "s_logit_token_index"}, {})
            dev = self.staging.upload(arrays)
            self.h2d_bytes += self.staging.last_words * 4
            hidden = self._run_model(model_id, p, dev, None)
        self.pp_microbatch_steps += 1
        return dev, hidden

    def _logits(self, model_id: int, hidden: torch.Tensor, rows: torch.Tensor, n_rows: Optional[int] = None
                ) -> torch.Tensor:
        """Logits of the selected rows on the rank that hosts the engine. With pipeline stages the
        last stage computes them and returns them to rank 0 (reference: ``SendFromLastGroupToWorker0``,
        ``cpp/multi_gpu/builtin.cc:27-87``)."""
        model = self.models[model_id]
        if not self._pipeline(model_id):
            return model.logits(hidden, rows)
        out = torch.empty(int(rows.numel()) if n_rows is None else int(n_rows), model.cfg.vocab_size,
                          dtype=torch.float32, device=self.device)
        self.comm.recv_logits_from_last_stage(out)
        return out

    def _process_logits(self, logits: torch.Tensor, dev: Dict[str, torch.Tensor], sp: dict) -> None:
        n = logits.shape[0]
        if dev["s_bias_row"].numel():
            ops.apply_logit_bias(logits, dev["s_bias_row"], dev["s_bias_token"], dev["s_bias_value"])
        if dev["s_pen_row"].numel():
            ops.apply_penalty(logits, dev["s_pen_row"], dev["s_pen_token"], dev["s_pen_count"],
                              dev["s_penalties"].view(n, 3))
        if dev["s_mask_rows"].numel():
            words = (logits.shape[1] + 31) // 32
            ops.apply_bitmask(logits, dev["s_mask_rows"], dev["s_mask_bits"].view(-1, words))

    @staticmethod
    def _is_plain_greedy(sp: dict) -> bool:
        return (len(sp["temperature"]) > 0 and float(np.max(sp["temperature"])) < 1e-5
                and sp["num_top_logprobs"] == 0 and len(sp["pen_row"]) == 0 and len(sp["bias_row"]) == 0
                and len(sp["mask_rows"]) == 0 and len(sp["prob_slots"]) == 0)

    def _ensure_draft_storage(self, max_slot: int) -> None:
        need = max(max_slot + 1, self.max_draft_slots)
        if self.draft_probs is None or self.draft_probs.shape[0] < need:
            new = torch.zeros(need, self.vocab, dtype=torch.float32, device=self.device)
            if self.draft_probs is not None:
                new[: self.draft_probs.shape[0]] = self.draft_probs
            self.draft_probs = new

    # ------------------------------------------------------------------ backend interface
    def forward_sample(self, model_id: int, plan: dict, token_ids: np.ndarray,
                       embed_handles: Optional[np.ndarray], sp: dict) -> Optional[dict]:
        if not self._nvtx:
            return self._forward_sample(model_id, plan, token_ids, embed_handles, sp)
        # NVTX range per model call (reference: NVTXScopedRange around every action, cpp/serve/model.cc:88,262)
        torch.cuda.nvtx.range_push(f"forward_sample model={model_id} tokens={len(token_ids)} rows={len(sp['logit_token_index'])}")
        try:
            return self._forward_sample(model_id, plan, token_ids, embed_handles, sp)
        finally:
            torch.cuda.nvtx.range_pop()

    def _forward_sample(self, model_id: int, plan: dict, token_ids: np.ndarray,
                        embed_handles: Optional[np.ndarray], sp: dict) -> Optional[dict]:
        self._enter()
        ht, clock = self.host_times, time.perf_counter
        t0 = clock()
        n_rows = len(sp["logit_token_index"])
        if self.spec_heads:
            self._fork_features(plan)
        parts = self._pipeline_parts(model_id, plan, token_ids, embed_handles, sp)
        if parts is not None:
            # the parts were packed, announced and launched one after the other; `dev` holds the last one's
            # arrays, with the sampling parameters of every row
            dev, hidden = parts
            t1 = t2 = t3 = clock()
        else:
            arrays = self._pack(plan, token_ids, sp, model_id)
            t1 = clock()
            if self.comm is not None and self.spec_heads.get(model_id) != "medusa":
                self.comm.broadcast_step("forward", model_id,
                                         {k: v for k, v in arrays.items()
                                          if not k.startswith("s_") or k == "s_logit_token_index"}, {})
            t2 = clock()
            dev = self.staging.upload(arrays)
            self.h2d_bytes += self.staging.last_words * 4
            t3 = clock()
            if model_id in self.spec_heads:
                logits = self._forward_spec_head(model_id, plan, dev, n_rows)
                if logits is None:
                    return None
                return self._sample(logits, dev, sp, n_rows)
            hidden = self._run_model(model_id, plan, dev, embed_handles)
        t4 = clock()
        ht["pack"] += t1 - t0
        ht["broadcast"] += t2 - t1
        ht["upload"] += t3 - t2
        ht["forward"] += t4 - t3
        ht["calls"] += 1
        if self.spec_heads and model_id == 0:
            self._remember_features(plan, self.models[0].final_features(hidden), None)
        if n_rows == 0:
            return None
        logits = self._logits(model_id, hidden, dev["s_logit_token_index"], n_rows)
        if self._is_plain_greedy(sp):
            tokens = ops.argmax(logits)
            t5 = clock()
            tok = tokens.cpu().numpy()
            ht["logits_sample"] += t5 - t4
            ht["readback"] += clock() - t5
            self.d2h_bytes += tok.nbytes
            return {"tokens": tok, "probs": np.ones(n_rows, dtype=np.float32)}
        return self._sample(logits, dev, sp, n_rows)

    # ------------------------------------------------------------------ deferred-read decode steps
    def _feed_tokens(self, model_id: int, dev: Dict[str, torch.Tensor]) -> None:
        """``token_ids[i] = last_tokens[token_src[i]]`` where ``token_src[i] >= 0``: the tokens the previous
        launched step sampled become this step's inputs without visiting the host."""
        last = self._last_tokens.get(model_id)
        if last is None:
            raise RuntimeError("a decode step refers to the tokens of a step this executor never launched")
        tok, src = dev["token_ids"], dev["token_src"]
        if tok.is_cuda:
            from ..ops._lib import check, lib, ptr, stream_ptr  # pylint: disable=import-outside-toplevel

            rc = lib().mlcb_token_feed(ptr(tok), ptr(src), ptr(last), ctypes.c_int(tok.numel()),
                                       ctypes.c_int(last.numel()), ptr(ops.status_word(self.device)), stream_ptr())
            check(rc, "mlcb_token_feed")
        else:
            pick = src >= 0
            tok[pick] = last[src[pick].long()]

    def _readback(self, name: str, t: torch.Tensor) -> torch.Tensor:
        """Queue a device -> pinned host copy of ``t``; the buffers alternate between two steps."""
        if not t.is_cuda:
            return t
        bufs = self._readback_bufs[self._readback_turn]
        buf = bufs.get(name)
        if buf is None or buf.numel() < t.numel() or buf.dtype != t.dtype:
            buf = bufs[name] = torch.empty(max(t.numel(), 1024), dtype=t.dtype, pin_memory=True)
        out = buf[: t.numel()].view(t.shape)
        out.copy_(t, non_blocking=True)
        return out

    def forward_sample_launch(self, model_id: int, plan: dict, token_ids: np.ndarray, token_src: np.ndarray,
                              sp: dict) -> bool:
        """Queue one decode step and return without reading its result (``forward_sample_wait`` does).
        Returns False, having done nothing, for steps that need the synchronous path."""
        model = self.models[model_id]
        n_rows = len(sp["logit_token_index"])
        if (model_id in self.spec_heads or self._pipeline(model_id) or getattr(model, "stateful", False)
                or n_rows == 0 or len(sp["prob_slots"]) or len(sp["pen_row"]) or len(sp["mask_rows"])
                or len(self._pending) >= 2):
            return False
        self._enter()
        ht, clock = self.host_times, time.perf_counter
        t0 = clock()
        arrays = self._pack(plan, token_ids, sp, model_id)
        src = np.ascontiguousarray(token_src, dtype=np.int32)
        pad = int(arrays["token_ids"].size) - int(src.size)  # stand-in sequences of a padded decode batch
        arrays["token_src"] = np.concatenate([src, np.full(pad, -1, np.int32)]) if pad > 0 else src
        feed = bool((src >= 0).any())
        t1 = clock()
        if self.comm is not None:
            self.comm.broadcast_step("forward_async", model_id,
                                     {k: v for k, v in arrays.items()
                                      if not k.startswith("s_") or k == "s_logit_token_index"}, {})
        t2 = clock()
        dev = self.staging.upload(arrays)
        self.h2d_bytes += self.staging.last_words * 4
        t3 = clock()
        if feed:
            self._feed_tokens(model_id, dev)
        hidden = self._run_model(model_id, plan, dev, None)
        t4 = clock()
        logits = self._logits(model_id, hidden, dev["s_logit_token_index"])
        res: Dict[str, torch.Tensor] = {}
        if self._is_plain_greedy(sp):
            tokens = ops.argmax(logits)
        else:
            self._process_logits(logits, dev, sp)
            probs = ops.softmax_temperature(logits, dev["s_temperature"])
            top_k = dev["s_top_k"] if int(np.max(sp["top_k"])) > 0 else None
            tokens, tprobs = ops.sample(probs, None, dev["s_uniform"], dev["s_top_p"], top_k)
            tokens = tokens.to(torch.int32)
            k = int(sp["num_top_logprobs"])
            if k > 0:
                _, tp, ti = ops.take_probs(probs, None, tokens, k)
                res["top_probs"] = self._readback("top_probs", tp.reshape(-1).float())
                res["top_tokens"] = self._readback("top_tokens", ti.reshape(-1).to(torch.int32))
                # logprobs are reported on the unrenormalised distribution
                tprobs = probs[torch.arange(n_rows, device=probs.device), tokens.long()]
            res["probs"] = self._readback("probs", tprobs.float())
        self._last_tokens[model_id] = tokens
        if self.comm is not None:
            self.comm.broadcast_tokens(tokens)
        res["tokens"] = self._readback("tokens", tokens)
        event = None
        if tokens.is_cuda:
            event = torch.cuda.Event()
            event.record()
        self._readback_turn ^= 1
        self._pending.append({"model": model_id, "res": res, "event": event, "rows": n_rows})
        t5 = clock()
        ht["pack"] += t1 - t0
        ht["broadcast"] += t2 - t1
        ht["upload"] += t3 - t2
        ht["forward"] += t4 - t3
        ht["logits_sample"] += t5 - t4
        ht["calls"] += 1
        return True

    def forward_sample_wait(self, model_id: int) -> dict:
        """Result of the oldest launched step that has not been read."""
        if not self._pending:
            raise RuntimeError("no launched decode step to wait for")
        t0 = time.perf_counter()
        item = self._pending.popleft()
        if item["event"] is not None:
            item["event"].synchronize()
        out = {k: np.array(v.numpy() if not v.is_cuda else v.cpu().numpy()) for k, v in item["res"].items()}
        if "probs" not in out:
            out["probs"] = np.ones(item["rows"], dtype=np.float32)
        self.d2h_bytes += sum(v.nbytes for k, v in out.items() if k in item["res"])
        self.host_times["readback"] += time.perf_counter() - t0
        return out

    def _sample(self, logits: torch.Tensor, dev: Dict[str, torch.Tensor], sp: dict, n_rows: int) -> dict:
        """Logit processing, softmax, sampling and read-back of one row per entry of ``sp``."""
        self._process_logits(logits, dev, sp)
        probs = ops.softmax_temperature(logits, dev["s_temperature"])
        if len(sp["prob_slots"]):
            # draft model: the verifier needs the distribution the token was actually drawn from
            if float(np.min(sp["top_p"])) < 1.0:
                ops.renorm_top_p(probs, None, dev["s_top_p"])
            self._ensure_draft_storage(int(np.max(sp["prob_slots"])))
            ops.row_scatter(self.draft_probs, dev["s_prob_slots"], probs)
            ones = torch.ones_like(dev["s_top_p"])
            tokens, tprobs = ops.sample(probs, None, dev["s_uniform"], ones, None)
        else:
            top_k = dev["s_top_k"] if int(np.max(sp["top_k"])) > 0 else None
            tokens, tprobs = ops.sample(probs, None, dev["s_uniform"], dev["s_top_p"], top_k)
        out = {}
        k = int(sp["num_top_logprobs"])
        if k > 0:
            rank = probs
            if len(sp["prob_slots"]) and float(np.min(sp["temperature"])) < 1e-5:
                # children of a draft tree are the draft's k best tokens; under greedy sampling the sampling
                # distribution is one-hot and ranks nothing below the first, so those rows are ranked by the
                # plain softmax (the stored draft distribution stays the one-hot one: the verifier accepts a
                # lower-ranked child exactly when the target's arg-max is that token)
                temp = dev["s_temperature"]
                rank = ops.softmax_temperature(logits, torch.where(temp < 1e-5, torch.ones_like(temp), temp))
            _, tp, ti = ops.take_probs(rank, None, tokens if tokens.device == probs.device
                                       else tokens.to(probs.device), k)
            out["top_probs"] = tp.reshape(-1).float().cpu().numpy()
            out["top_tokens"] = ti.reshape(-1).to(torch.int32).cpu().numpy()
            # logprobs are reported on the unrenormalised distribution
            sel = probs[torch.arange(n_rows, device=probs.device), tokens.long().to(probs.device)]
            tprobs = sel
        out["tokens"] = tokens.to(torch.int32).cpu().numpy()
        out["probs"] = tprobs.float().cpu().numpy()
        self.d2h_bytes += out["tokens"].nbytes + out["probs"].nbytes
        return out

    # ------------------------------------------------------------------ EAGLE / Medusa draft heads
    def _fork_features(self, plan: dict) -> None:
        """Forks reported by a plan (of the target's or of the head's KV manager) carry the features along."""
        for parent, child in np.asarray(plan.get("seq_forks", ()), dtype=np.int64).reshape(-1, 2).tolist():
            self.features.fork(int(parent), int(child))

    def _remember_features(self, plan: dict, feats: torch.Tensor, rows_of_seq: Optional[List[List[int]]]) -> None:
        """Store the target's features of this forward: all rows of every sequence (prefill, decode), or
        only ``rows_of_seq[i]`` (verification: the root and the accepted nodes, which sit at consecutive
        positions)."""
        qi = np.asarray(plan["q_indptr"])
        pos = np.asarray(plan["positions"])
        for i, sid in enumerate(np.asarray(plan["seq_ids"]).tolist()):
            a, b = int(qi[i]), int(qi[i + 1])
            if b <= a:
                continue
            if rows_of_seq is None:
                self.features.put(int(sid), int(pos[a]), feats[a:b])
            else:
                idx = torch.as_tensor(rows_of_seq[i], dtype=torch.long, device=feats.device)
                self.features.put(int(sid), int(pos[a]), feats.index_select(0, idx))

    def _forward_spec_head(self, model_id: int, plan: dict, dev: Dict[str, torch.Tensor], n_rows: int
                           ) -> Optional[torch.Tensor]:
        """Forward of a feature-fed draft head over the tokens of ``plan``; returns the logits of the
        sample rows (None when the call only advances the head's state, i.e. its prefill)."""
        kind = self.spec_heads[model_id]
        head, target = self.models[model_id], self.models[0]
        qi = np.asarray(plan["q_indptr"])
        pos = np.asarray(plan["positions"])
        ids = [int(x) for x in np.asarray(plan["seq_ids"]).tolist()]
        hsz = target.cfg.hidden_size
        if kind == "medusa":
            # no state of its own: draft round r uses head r on the newest true feature
            if n_rows == 0:
                return None
            heads = int(head.cfg.extra["medusa"]["num_heads"])
            feats = torch.zeros(len(ids), hsz, dtype=target.dtype, device=self.device)
            which = np.zeros(len(ids), dtype=np.int64)
            for i, sid in enumerate(ids):
                s0, t = self.features.span(sid)
                if t is not None:
                    feats[i] = t[-1]
                    which[i] = min(max(int(pos[int(qi[i + 1]) - 1]) - (s0 + t.shape[0]), 0), heads - 1)
            logits = torch.empty(len(ids), head.cfg.vocab_size, dtype=torch.float32, device=self.device)
            for j in sorted(set(which.tolist())):
                sel = torch.as_tensor(np.nonzero(which == j)[0], dtype=torch.long, device=self.device)
                logits[sel] = head.medusa_logits(feats.index_select(0, sel), int(j))
            if n_rows != len(ids):
                # draft tree: every leaf of a sequence asks for the distribution of the same head (a Medusa
                # head does not see the drafted tokens), so the sequence's row is repeated for its leaves
                seq_of_row = dev["q_seq"].index_select(0, dev["s_logit_token_index"].long()).long()
                logits = logits.index_select(0, seq_of_row)
            return logits
        # ---- EAGLE: token at position p is fused with the feature of position p - 1
        if dev["page_copies"].numel():
            head.copy_pages(dev["page_copies"])
        x = head.embed(dev["token_ids"])
        prev = torch.zeros(x.shape[0], hsz, dtype=x.dtype, device=self.device)
        all_true = []
        masks = np.asarray(plan["tree_mask"]).astype(np.uint64) if len(plan["tree_mask"]) else None
        for i, sid in enumerate(ids):
            a, b = int(qi[i]), int(qi[i + 1])
            if b <= a:
                all_true.append(False)
                continue
            if masks is not None:
                # a draft tree fed as one chunk (node j = row a + j, ancestors in its mask): a child of the root
                # continues from the head's output at the last committed token, any other node from the output
                # the head gave for its parent when the previous, smaller tree was fed
                own, old = self.features.pred.get(sid), self.features.tree.get(sid)
                for j in range(b - a):
                    below = int(masks[a + j]) & ((1 << j) - 1)
                    parent = below.bit_length() - 1
                    if parent < 0:
                        if own is not None and own[0] == int(pos[a + j]) - 1:
                            prev[a + j] = own[1].to(x.dtype)
                    elif old is not None and parent < old.shape[0]:
                        prev[a + j] = old[parent].to(x.dtype)
                all_true.append(False)
                continue
            s0, t = self.features.span(sid)
            first = int(pos[a]) - 1            # feature position wanted by row a
            covered = 0
            if t is not None:
                lo, hi = max(first, s0), min(first + (b - a), s0 + t.shape[0])
                if hi > lo:
                    prev[a + (lo - first): a + (hi - first)] = t[lo - s0: hi - s0].to(x.dtype)
                    covered = hi - lo
            own = self.features.pred.get(sid)
            if own is not None and first <= own[0] < first + (b - a) and (t is None or own[0] >= s0 + t.shape[0]):
                prev[a + (own[0] - first)] = own[1].to(x.dtype)
            all_true.append(covered == b - a)
        if self.comm is not None:
            self.comm.broadcast_tokens(prev)  # the other ranks fuse the same rows (see worker_step)
        x = head.fuse_embed_hidden(x, prev)
        h = head.forward(x, self._batch_info(dev, plan, head))
        for i, sid in enumerate(ids):
            a, b = int(qi[i]), int(qi[i + 1])
            if b <= a:
                continue
            if masks is not None:
                self.features.tree[sid] = h[a:b].detach().clone()  # the root's output (pred) stays as it is
                continue
            if all_true[i]:
                self.features.trim(sid, int(pos[b - 1]) - 1)
            self.features.pred[sid] = (int(pos[b - 1]), h[b - 1].detach().clone())
        if n_rows == 0:
            return None
        return target.head_logits(ops.row_gather(h, dev["s_logit_token_index"]))

    def forward_verify(self, model_id: int, plan: dict, token_ids: np.ndarray, vp: dict) -> dict:
        if self._nvtx:
            torch.cuda.nvtx.range_push(f"forward_verify model={model_id} tokens={len(token_ids)}")
            try:
                return self._forward_verify(model_id, plan, token_ids, vp)
            finally:
                torch.cuda.nvtx.range_pop()
        return self._forward_verify(model_id, plan, token_ids, vp)

    def _forward_verify(self, model_id: int, plan: dict, token_ids: np.ndarray, vp: dict) -> dict:
        self._enter()
        sp = vp["sampling"]
        if self.spec_heads:
            self._fork_features(plan)
        arrays = self._pack(plan, token_ids, sp, model_id)
        if self.comm is not None:
            self.comm.broadcast_step("forward", model_id,
                                     {k: v for k, v in arrays.items()
                                      if not k.startswith("s_") or k == "s_logit_token_index"}, {})
        dev = self.staging.upload(arrays)
        self.h2d_bytes += self.staging.last_words * 4
        hidden = self._run_model(model_id, plan, dev, None)
        feats = self.models[0].final_features(hidden) if (self.spec_heads and model_id == 0) else None
        logits = self._logits(model_id, hidden, dev["s_logit_token_index"])
        self._process_logits(logits, dev, sp)
        probs = ops.softmax_temperature(logits, dev["s_temperature"])
        if float(np.min(sp["top_p"])) < 1.0:
            ops.renorm_top_p(probs, None, dev["s_top_p"])
        top_k = np.asarray(sp["top_k"])
        if top_k.size and int(top_k.max()) > 0:
            # the verified distribution is the one plain decoding samples from: the k best of the top-p set
            for k in sorted(set(int(v) for v in top_k.tolist() if 0 < v < probs.shape[1])):
                rows = torch.from_numpy(np.nonzero(top_k == k)[0]).to(probs.device)
                sub = probs.index_select(0, rows)
                kth = torch.topk(sub, k, dim=-1).values[:, -1:]
                sub = torch.where(sub >= kth, sub, torch.zeros_like(sub))
                probs.index_copy_(0, rows, sub / sub.sum(dim=-1, keepdim=True).clamp_min(1e-30))
        # flat node table: row r of `probs` is node r; roots carry no draft token
        node_indptr = np.asarray(vp["node_indptr"])
        nseq = len(node_indptr) - 1
        total_rows = probs.shape[0]
        first_child = np.full(total_rows, -1, dtype=np.int32)
        next_sibling = np.full(total_rows, -1, dtype=np.int32)
        draft_tok = np.zeros(total_rows, dtype=np.int32)
        uniform = np.zeros(total_rows, dtype=np.float32)
        slot_of_row = np.zeros(total_rows, dtype=np.int32)
        parent_row = np.full(total_rows, -1, dtype=np.int32)
        roots = np.zeros(nseq, dtype=np.int32)
        parents = np.asarray(vp["parents"])
        row = 0
        for s in range(nseq):
            root = row
            roots[s] = root
            nb, ne = int(node_indptr[s]), int(node_indptr[s + 1])
            last_child: Dict[int, int] = {}
            for j in range(nb, ne):
                r = root + 1 + (j - nb)
                p = root if parents[j] < 0 else root + 1 + int(parents[j])
                parent_row[r] = p
                if p in last_child:
                    next_sibling[last_child[p]] = r
                else:
                    first_child[p] = r
                last_child[p] = r
                draft_tok[r] = vp["draft_tokens"][j]
                uniform[r] = vp["uniform"][j]
                slot_of_row[r] = vp["draft_prob_slots"][j]
            row += 1 + (ne - nb)
        d = self.device
        self._ensure_draft_storage(int(slot_of_row.max()) if total_rows else 0)
        if bool((next_sibling >= 0).any()):
            # A draft tree: its children are the draft's k best tokens, chosen, not drawn. The acceptance rule
            # min(1, p / q) is only unbiased for candidates DRAWN from q; for chosen candidates the draft
            # distribution of a child is the point mass on its token: accept with probability p(token), on a
            # rejection drop the token from p and renormalise. (Under greedy sampling both rules coincide.)
            draft_rows = torch.zeros(total_rows, probs.shape[1], dtype=probs.dtype, device=d)
            draft_rows.scatter_(1, torch.from_numpy(draft_tok.astype(np.int64)).to(d).unsqueeze(1), 1.0)
        else:
            draft_rows = ops.row_gather(self.draft_probs, torch.from_numpy(slot_of_row).to(d))
        parent_ptr = torch.from_numpy(roots.copy()).to(d)
        ops.verify_tree(draft_rows, torch.from_numpy(draft_tok).to(d), probs,
                        torch.from_numpy(first_child).to(d), torch.from_numpy(next_sibling).to(d),
                        torch.from_numpy(uniform).to(d), parent_ptr)
        fin_u = torch.from_numpy(np.asarray(vp["final_uniform"], dtype=np.float32)).to(d)
        tokens, tprobs = ops.sample(probs, parent_ptr, fin_u, torch.ones_like(fin_u), None)
        last = parent_ptr.cpu().numpy()
        accepted_indptr = [0]
        accepted_nodes: List[int] = []
        for s in range(nseq):
            path = []
            r = int(last[s])
            while r != roots[s]:
                path.append(r - roots[s] - 1)
                r = int(parent_row[r])
            accepted_nodes.extend(reversed(path))
            accepted_indptr.append(len(accepted_nodes))
        if feats is not None:
            # the draft head continues from the true features of the root and of the accepted nodes
            qi = np.asarray(plan["q_indptr"])
            keep = [[int(qi[s_])] + [int(qi[s_]) + 1 + n for n in accepted_nodes[accepted_indptr[s_]:accepted_indptr[s_ + 1]]]
                    for s_ in range(nseq)]
            self._remember_features(plan, feats, keep)
        out = {"accepted_indptr": np.asarray(accepted_indptr, dtype=np.int32),
               "accepted_nodes": np.asarray(accepted_nodes, dtype=np.int32),
               "final_tokens": tokens.to(torch.int32).cpu().numpy(),
               "final_probs": tprobs.float().cpu().numpy()}
        if bool(vp.get("want_logprobs", False)) or int(sp["num_top_logprobs"]) > 0:
            # what is reported for a committed token is the TARGET's probability of it (on the distribution before
            # top-p / top-k and before the residual updates of the verification), not the draft's: recompute the
            # rows that produced the accepted tokens and the final ones from the processed logits
            src_rows, toks = [], []
            for s_ in range(nseq):
                for n in accepted_nodes[accepted_indptr[s_]:accepted_indptr[s_ + 1]]:
                    r = int(roots[s_]) + 1 + int(n)
                    src_rows.append(int(parent_row[r]))
                    toks.append(int(draft_tok[r]))
            src_rows += [int(v) for v in last.tolist()]
            toks += [int(v) for v in out["final_tokens"].tolist()]
            sel = torch.as_tensor(src_rows, dtype=torch.long, device=d)
            base = ops.softmax_temperature(logits.index_select(0, sel).contiguous(),
                                           dev["s_temperature"].index_select(0, sel).contiguous())
            tok_t = torch.as_tensor(toks, dtype=torch.long, device=d)
            own = base.gather(1, tok_t.unsqueeze(1)).squeeze(1).float().cpu().numpy()
            n_acc = len(accepted_nodes)
            out["accepted_probs"] = own[:n_acc]
            out["final_probs"] = own[n_acc:]
            k_top = int(sp["num_top_logprobs"])
            if k_top > 0:
                tp, ti = torch.topk(base, k_top, dim=-1)
                out["top_probs"] = tp.reshape(-1).float().cpu().numpy()
                out["top_tokens"] = ti.reshape(-1).to(torch.int32).cpu().numpy()
                out["num_top"] = k_top
        return out

    def move_kv_tokens(self, model_id: int, moves: np.ndarray) -> None:
        self._enter()
        if self.comm is not None:
            self.comm.broadcast_step("move", model_id, {"moves": np.ascontiguousarray(moves, dtype=np.int32)}, {})
        self.models[model_id].move_tokens(torch.from_numpy(np.ascontiguousarray(moves, dtype=np.int32)).to(self.device))

    # ------------------------------------------------------------------ disaggregated serving
    def apply_page_copies(self, model_id: int, copies: np.ndarray) -> None:
        """Copy-on-write page copies of a KV reservation that is not followed by a forward call."""
        self._enter()
        if self.comm is not None and self.comm.world_size > 1:
            raise RuntimeError("disaggregated serving supports single-GPU endpoints only")
        pairs = torch.from_numpy(np.ascontiguousarray(copies, dtype=np.int32)).to(self.device)
        self.models[model_id].copy_pages(pairs)

    def kv_export(self, model_id: int = 0) -> dict:
        """Fixed-format description of this engine's KV pool that a peer engine can write into: an
        in-process registry key (engines sharing a process, CPU tests) plus, on GPUs, the 64 raw bytes
        of a CUDA IPC memory handle and the pool's offset inside that allocation (engines in different
        processes of one NVLink box). See ``serve/kv_handoff.py`` for the schema."""
        import uuid  # pylint: disable=import-outside-toplevel

        from . import kv_handoff  # pylint: disable=import-outside-toplevel

        pool = self.models[model_id].kv_pages
        key = getattr(self, "_kv_export_key", None)
        if key is None:
            key = self._kv_export_key = uuid.uuid4().hex
            _LOCAL_KV_POOLS[key] = pool
        handle, offset = b"", 0
        if pool.is_cuda:
            from ..ops._lib import check, lib  # pylint: disable=import-outside-toplevel

            buf = (ctypes.c_ubyte * 64)()
            off, size = ctypes.c_longlong(0), ctypes.c_longlong(0)
            with torch.cuda.device(pool.device):
                rc = lib().mlcb_ipc_export(ctypes.c_void_p(pool.data_ptr()), buf, ctypes.byref(off), ctypes.byref(size))
            check(rc, "mlcb_ipc_export")
            handle, offset = bytes(buf), int(off.value)
        return kv_handoff.pool_descriptor(key, list(pool.shape), str(pool.dtype),
                                          pool.device.index if pool.is_cuda else -1, handle, offset)

    def _peer_pool(self, desc: dict):
        """(tensor or None, device pointer, pages) of the receiver's pool named by a verified descriptor."""
        from . import kv_handoff  # pylint: disable=import-outside-toplevel

        if desc["pid"] == os.getpid() and desc["key"] in _LOCAL_KV_POOLS:
            pool = _LOCAL_KV_POOLS[desc["key"]]
            if list(pool.shape) != desc["shape"] or str(pool.dtype) != desc["dtype"]:
                raise kv_handoff.HandoffError("pool descriptor does not match the registered pool")
            return pool, (pool.data_ptr() if pool.is_cuda else 0)
        cache = self.__dict__.setdefault("_peer_pools", {})
        entry = cache.get(desc["key"])
        if entry is None:
            if len(desc["handle"]) != 64 or not self.device.type == "cuda":
                raise kv_handoff.HandoffError("the receiving engine did not export a device memory handle")
            from ..ops._lib import check, lib  # pylint: disable=import-outside-toplevel

            base, mapped = ctypes.c_void_p(0), ctypes.c_longlong(0)
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(desc["handle"])
            with torch.cuda.device(self.device):
                rc = lib().mlcb_ipc_open(buf, ctypes.byref(base), ctypes.byref(mapped))
            check(rc, "mlcb_ipc_open (is the receiving engine on this NVLink box?)")
            entry = cache[desc["key"]] = (int(base.value), int(mapped.value))
        base, mapped = entry
        need = int(np.prod(desc["shape"], dtype=np.int64)) * torch.empty(0, dtype=_KV_DTYPES[desc["dtype"]]).element_size()
        if desc["offset"] + need > mapped:
            raise kv_handoff.HandoffError("pool descriptor claims more memory than the mapped allocation holds")
        return None, base + desc["offset"]

    def send_kv(self, model_id: int, src_slots: np.ndarray, metadata: str) -> None:
        """Prefill side of the hand-off: copy the KV rows at ``src_slots`` into the receiver's slots.
        ``metadata`` is the signed payload of the receiver's ``prep_recv`` step
        (``kv_handoff.encode_payload``); it is verified and range-checked before anything is launched."""
        self._enter()
        from . import kv_handoff  # pylint: disable=import-outside-toplevel

        meta = kv_handoff.decode_payload(metadata)
        pool_desc = meta["pool"]
        dst_slots = np.asarray(meta["slots"], dtype=np.int64)
        src_slots = np.ascontiguousarray(src_slots, dtype=np.int64)
        if len(dst_slots) != len(src_slots):
            raise kv_handoff.HandoffError(
                f"KV hand-off size mismatch: {len(src_slots)} rows to send, {len(dst_slots)} reserved")
        src = self.models[model_id].kv_pages
        dshape = pool_desc["shape"]
        if dshape[2:] != list(src.shape[2:]) or dshape[0] != src.shape[0] or pool_desc["dtype"] != str(src.dtype):
            raise kv_handoff.HandoffError("the two engines do not hold the same model / KV layout")
        page = src.shape[4]
        kv_handoff.check_slots(src_slots, src.shape[1], page, "source")
        kv_handoff.check_slots(dst_slots, dshape[1], page, "destination")
        dst, dst_ptr = self._peer_pool(pool_desc)
        if not src.is_cuda:
            if dst is None:
                raise kv_handoff.HandoffError("a CPU engine can only hand KV to an engine of its own process")
            s, d = torch.from_numpy(src_slots), torch.from_numpy(dst_slots)
            dst[:, d // page, :, :, d % page, :] = src[:, s // page, :, :, s % page, :]
            return
        from ..ops._lib import check, lib, ptr, status_word, stream_ptr  # pylint: disable=import-outside-toplevel

        if src.shape[2] != 2:
            # the slot-copy kernel addresses pages as [K | V] x heads; the compressed latent cache has one row
            raise kv_handoff.HandoffError("the compressed latent cache (mla_cache=latent) cannot be handed off "
                                          "between GPU engines; use the expanded cache on disaggregated endpoints")
        if pool_desc["device"] != src.device.index and dst is not None:
            rc = lib().mlcb_enable_peer_access(ctypes.c_int(src.device.index), ctypes.c_int(pool_desc["device"]))
            check(rc, f"peer access from GPU {src.device.index} to GPU {pool_desc['device']}")
        ss = torch.from_numpy(src_slots.astype(np.int32)).to(self.device)
        ds = torch.from_numpy(dst_slots.astype(np.int32)).to(self.device)
        es = src.element_size()
        dst_layer_stride = int(np.prod(dshape[1:], dtype=np.int64))
        rc = lib().mlcb_kv_slot_copy(
            ptr(src), ctypes.c_void_p(dst_ptr), ptr(ss), ptr(ds), ctypes.c_int(len(src_slots)),
            ctypes.c_int(src.shape[0]), ctypes.c_longlong(src.stride(0) * es), ctypes.c_longlong(dst_layer_stride * es),
            ctypes.c_int(src.shape[3]), ctypes.c_int(page), ctypes.c_int(src.shape[5] * es),
            ctypes.c_int(src.shape[1]), ctypes.c_int(dshape[1]), ptr(status_word(self.device)), stream_ptr())
        check(rc, "mlcb_kv_slot_copy")
        torch.cuda.synchronize(self.device)  # the receiver may start as soon as this call returns

    # ------------------------------------------------------------------ worker side (rank > 0)
    def worker_step(self, op: str, model_id: int, arrays: Dict[str, np.ndarray], layout) -> None:
        """Mirror of the rank-0 calls on the other tensor-parallel ranks: same forward, no sampling."""
        self._enter()
        if op == "move":
            self.models[model_id].move_tokens(torch.from_numpy(arrays["moves"]).to(self.device))
            return
        dev = self.staging.upload(arrays)
        plan = {k: arrays[k] for k in _INT_KEYS}
        plan["tree_mask"] = arrays["tree_mask"]
        plan["max_seq_len"] = int(arrays["seq_lens"].max()) if arrays["seq_lens"].size else 0
        if "seq_ids" in arrays:
            plan["seq_ids"] = arrays["seq_ids"]
            plan["seq_forks"] = arrays.get("seq_forks", np.zeros(0, dtype=np.int32))
        if op == "forward_async":
            # deferred-read decode step: inputs may be the tokens rank 0 sampled in the step before, and
            # this step's tokens arrive the same way (device to device) once rank 0 has sampled them
            if bool((arrays["token_src"] >= 0).any()):
                self._feed_tokens(model_id, dev)
            self._run_model(model_id, plan, dev, None)
            tokens = torch.empty(int(arrays["s_logit_token_index"].size), dtype=torch.int32, device=self.device)
            self.comm.broadcast_tokens(tokens)
            self._last_tokens[model_id] = tokens
            return
        if self.spec_heads.get(model_id) == "eagle":
            # this rank's shard of the draft head: the feature rows come from rank 0, the output stays here
            head = self.models[model_id]
            if dev["page_copies"].numel():
                head.copy_pages(dev["page_copies"])
            x = head.embed(dev["token_ids"])
            prev = torch.empty(x.shape[0], self.models[0].cfg.hidden_size, dtype=x.dtype, device=self.device)
            self.comm.broadcast_tokens(prev)
            head.forward(head.fuse_embed_hidden(x, prev), self._batch_info(dev, plan, head))
            return
        hidden = self._run_model(model_id, plan, dev, None)
        model = self.models[model_id]
        if self._pipeline(model_id) and model.last_stage and self.comm.tp_rank == 0:
            rows = dev.get("s_logit_token_index")
            if rows is not None and rows.numel():
                self._part_logits.append(model.logits(hidden, rows))
            if op == "forward" and self._part_logits:
                # one message for the rows of every part of the step
                out = self._part_logits[0] if len(self._part_logits) == 1 else torch.cat(self._part_logits)
                self._part_logits = []
                self.comm.send_logits_to_rank0(out)
