#include "engine.h"

#include <algorithm>
#include <cstdlib>
#include <cmath>
#include <sstream>
#include <stdexcept>

namespace mlcb {

namespace {

using json::Object;
using json::Value;

struct EntryRef {
  RequestState* rs;
  int idx;
  RequestStateEntry& e() const { return rs->entries[idx]; }
  bool operator==(const EntryRef& o) const { return rs == o.rs && idx == o.idx; }
};

class IdManager {
 public:
  int64_t Get() {
    if (!free_.empty()) {
      int64_t id = free_.back();
      free_.pop_back();
      return id;
    }
    return next_++;
  }
  void Recycle(int64_t id) { free_.push_back(id); }
  void Reset() {
    free_.clear();
    next_ = 0;
  }

 private:
  std::vector<int64_t> free_;
  int64_t next_ = 0;
};

// Ref-counted slots of the on-device draft-probability storage.
class SlotManager {
 public:
  explicit SlotManager(int n = 0) { Resize(n); }
  void Resize(int n) {
    free_.clear();
    for (int i = n - 1; i >= 0; --i) free_.push_back(i);
  }
  int Alloc() {
    if (free_.empty()) throw std::runtime_error("draft token workspace exhausted");
    int s = free_.back();
    free_.pop_back();
    return s;
  }
  void Free(int s) { free_.push_back(s); }

 private:
  std::vector<int> free_;
};

std::string LogprobJSON(const Tokenizer* tok, const SampleResult& r) {
  auto one = [&](int32_t token, float prob) {
    Object o;
    const std::string& bytes = tok ? tok->TokenBytes(token) : std::string();
    o["token"] = tok ? tok->Decode({token}) : std::to_string(token);
    o["logprob"] = static_cast<double>(std::log(std::max(prob, 1e-30f)));
    json::Array b;
    for (unsigned char c : bytes) b.emplace_back(static_cast<int>(c));
    o["bytes"] = Value(std::move(b));
    return o;
  };
  Object o = one(r.token, r.prob);
  json::Array top;
  for (auto& p : r.top) top.emplace_back(one(p.first, p.second));
  o["top_logprobs"] = Value(std::move(top));
  return Value(std::move(o)).dump();
}

// ====================================================================== EngineImpl
class EngineImpl : public Engine {
 public:
  EngineImpl(EngineConfig config, std::vector<EngineModelInfo> models,
             std::shared_ptr<ModelBackend> backend, std::shared_ptr<const Tokenizer> tokenizer,
             std::shared_ptr<GrammarBackend> grammar, std::shared_ptr<EventTraceRecorder> trace,
             StreamCallback callback)
      : cfg_(std::move(config)), models_(std::move(models)), backend_(std::move(backend)),
        tok_(std::move(tokenizer)), grammar_(std::move(grammar)), trace_(std::move(trace)),
        callback_(std::move(callback)),
        prefix_cache_(cfg_.prefix_cache_mode == PrefixCacheMode::kRadix,
                      cfg_.prefix_cache_max_num_recycling_seqs,
                      [this](int64_t id) { this->OnPrefixCacheRemove(id); }) {
    if (models_.empty()) throw std::runtime_error("Engine: no model");
    const int64_t max_seqs = cfg_.max_num_sequence * 2 + cfg_.prefix_cache_max_num_recycling_seqs + 8;
    for (auto& m : models_)
      kv_.emplace_back(new KVManager(m.num_pages, cfg_.kv_cache_page_size, max_seqs));
    if (!models_[0].generation_defaults_json.empty()) {
      Value v = json::parse(models_[0].generation_defaults_json);
      if (v.is_object()) default_gen_ = GenerationConfig::DefaultsFromModelConfig(v.as_object());
    }
    spec_ = cfg_.speculative_mode != SpeculativeMode::kDisable && models_.size() > 1;
    if (const char* env = std::getenv("MLCB_PIPELINED_DECODE")) pipelined_decode_ = env[0] != '0';
    feature_fed_draft_ = cfg_.speculative_mode == SpeculativeMode::kEagle ||
                         cfg_.speculative_mode == SpeculativeMode::kMedusa;
    if (spec_) draft_slots_.Resize(static_cast<int>(cfg_.max_num_sequence) * DraftSlotsPerSequence());
    std::random_device rd;
    seed_rng_.seed(rd());
  }

  // ---------------------------------------------------------------- public API
  void SetStreamCallback(StreamCallback cb) override { callback_ = std::move(cb); }
  const GenerationConfig& DefaultGenerationConfig() const override { return default_gen_; }
  const EngineConfig& Config() const override { return cfg_; }
  bool Empty() const override { return states_.empty(); }
  std::string JSONMetrics() const override { return metrics_.AsJSON().dump(); }
  std::string DebugStats() const override {
    Object o;
    o["num_prefill_steps"] = num_prefill_steps_;
    o["num_decode_steps"] = num_decode_steps_;
    o["num_pipelined_decode_steps"] = num_pipelined_steps_;
    o["num_dropped_pipelined_tokens"] = num_dropped_tokens_;
    o["num_verify_steps"] = num_verify_steps_;
    o["num_preemptions"] = num_preemptions_;
    o["num_running"] = static_cast<int64_t>(running_.size());
    o["num_waiting"] = static_cast<int64_t>(waiting_.size());
    o["kv_available_pages"] = kv_[0]->NumAvailablePages();
    o["kv_total_sequence_length"] = kv_[0]->TotalSequenceLength();
    o["prefix_cache_recycling"] = prefix_cache_.NumRecycling();
    // host seconds spent per phase of decode steps (profiling aid)
    Object t;
    t["assemble"] = t_assemble_;
    t["plan"] = t_plan_;
    t["backend"] = t_backend_;
    t["commit"] = t_commit_;
    t["postprocess"] = t_post_;
    o["decode_host_seconds"] = Value(std::move(t));
    return Value(std::move(o)).dump();
  }

  void AddRequest(Request request) override {
    Trace(request.id, "request added to engine");
    auto rs = std::make_unique<RequestState>();
    rs->request = std::move(request);
    Request& req = rs->request;
    req.prompt_tokens = 0;
    for (auto& in : req.inputs) req.prompt_tokens += in.Length();
    rs->metrics.prompt_tokens = req.prompt_tokens;
    rs->metrics.add_time = NowSeconds();
    if (req.cfg.debug_config.special_request == SpecialRequestKind::kQueryEngineMetrics) {
      RequestStreamOutput out;
      out.request_id = req.id;
      out.group_delta_token_ids.resize(1);
      out.group_delta_logprob_json_strs.resize(1);
      out.group_finish_reason = {"stop"};
      out.group_extra_prefix_string = {""};
      Object usage;
      usage["prompt_tokens"] = 0;
      usage["completion_tokens"] = 0;
      usage["total_tokens"] = 0;
      usage["extra"] = metrics_.AsJSON();
      out.request_final_usage_json_str = Value(std::move(usage)).dump();
      Emit({std::move(out)});
      return;
    }
    const DisaggConfig& dc = req.cfg.debug_config.disagg_config;
    if (dc.kind == DisaggRequestKind::kStartGeneration && TakeOverReservedRequest(rs.get())) return;
    if (dc.kind == DisaggRequestKind::kRemoteSend) {
      // prefill [0, end) only; the single sampled token is discarded by the caller
      int64_t end = dc.kv_window_end.value_or(-1);
      if (end < 0) end += req.prompt_tokens;
      end = std::max<int64_t>(1, std::min<int64_t>(end, req.prompt_tokens));
      TruncateInputs(&req.inputs, end);
      req.prompt_tokens = end;
      req.cfg.max_tokens = 1;
      req.cfg.n = 1;
      req.cfg.debug_config.ignore_eos = true;
    }
    if (states_.count(req.id)) throw std::runtime_error("duplicate request id " + req.id);
    const int n = req.cfg.n;
    const int num_entries = n == 1 ? 1 : n + 1;
    rs->entries.resize(num_entries);
    const uint64_t base_seed = req.cfg.seed >= 0 ? static_cast<uint64_t>(req.cfg.seed) : seed_rng_();
    for (int i = 0; i < num_entries; ++i) {
      RequestStateEntry& e = rs->entries[i];
      e.mstates.resize(models_.size());
      e.rng.seed(base_seed + static_cast<uint64_t>(i) * 0x9E3779B97F4A7C15ull);
      e.stop_handler = std::make_unique<StopStrHandler>(req.cfg.stop_strs, tok_);
      if (i > 0) {
        e.parent_idx = 0;
        rs->entries[0].child_indices.push_back(i);
      }
    }
    for (size_t m = 0; m < models_.size(); ++m)
      for (auto& in : req.inputs) rs->entries[0].mstates[m].inputs.push_back(in);
    rs->num_unfinished = n;
    // requests longer than the engine can ever hold finish immediately with "length"
    if (req.prompt_tokens >= cfg_.max_single_sequence_length || req.prompt_tokens == 0) {
      RequestStreamOutput out;
      out.request_id = req.id;
      out.group_delta_token_ids.resize(n);
      out.group_delta_logprob_json_strs.resize(n);
      out.group_finish_reason.assign(n, "length");
      out.group_extra_prefix_string.assign(n, "");
      rs->metrics.finish_time = rs->metrics.prefill_end_time = NowSeconds();
      out.request_final_usage_json_str = rs->metrics.AsUsageJSON(true).dump();
      Emit({std::move(out)});
      return;
    }
    if (grammar_ && req.cfg.response_format.type == "json_object") {
      const std::string rf = req.cfg.response_format.AsJSON().dump();
      for (int i = (n == 1 ? 0 : 1); i < num_entries; ++i) rs->entries[i].grammar_handle = grammar_->Create(rf);
    }
    RequestState* raw = rs.get();
    states_[req.id] = std::move(rs);
    if (dc.kind == DisaggRequestKind::kPrepareReceive) {
      PrepareReceive(raw);
      return;
    }
    waiting_.push_back(raw);
  }

  // ---------------------------------------------------------------- disaggregated serving
  // (reference: engine_actions/disagg_prepare_recv.cc, disagg_remote_send.cc and the
  // start-generation handling of new_request_prefill.cc)
  static void TruncateInputs(std::vector<InputItem>* inputs, int64_t keep) {
    int64_t left = keep;
    std::vector<InputItem> out;
    for (auto& in : *inputs) {
      if (left <= 0) break;
      if (in.kind != 0) throw std::runtime_error("disaggregated requests take token inputs only");
      InputItem it = in;
      if (static_cast<int64_t>(it.tokens.size()) > left) it.tokens.resize(left);
      left -= static_cast<int64_t>(it.tokens.size());
      out.push_back(std::move(it));
    }
    *inputs = std::move(out);
  }

  static std::vector<int32_t> AllTokens(const Request& req) {
    std::vector<int32_t> t;
    for (auto& in : req.inputs) t.insert(t.end(), in.tokens.begin(), in.tokens.end());
    return t;
  }

  // Decode side, step 1: match the prompt against the prefix cache, reserve KV entries for
  // [matched, end) and report where a sender may write them. The request then waits (outside the
  // scheduling queues) for its start-generation step.
  void PrepareReceive(RequestState* rs) {
    Request& req = rs->request;
    const DisaggConfig& dc = req.cfg.debug_config.disagg_config;
    try {
      if (req.cfg.n != 1) throw std::runtime_error("disaggregated requests must have n == 1");
      if (kv_.size() != 1) throw std::runtime_error("disaggregated serving does not combine with draft models");
      if (cfg_.sliding_window_size > 0) throw std::runtime_error("disaggregated serving needs a full KV cache");
      int64_t end = dc.kv_window_end.value_or(-1);
      if (end < 0) end += req.prompt_tokens;
      end = std::max<int64_t>(0, std::min<int64_t>(end, req.prompt_tokens - 1));  // the last token stays local
      std::vector<int32_t> tokens = AllTokens(req);
      RequestStateEntry& e = rs->entries[0];
      ModelState& ms = e.mstates[0];
      // match on the part that will be received
      ms.inputs.clear();
      InputItem head;
      head.tokens.assign(tokens.begin(), tokens.begin() + end);
      if (end > 0) ms.inputs.push_back(std::move(head));
      if (NumActiveSequences() + 1 > cfg_.max_num_sequence) throw std::runtime_error("too many sequences");
      MatchPrefixAndCreateSequence({rs, 0});
      const int64_t matched = ms.num_prefilled_tokens;
      const int64_t need = end - matched;
      ForwardPlan plan;
      if (need > 0) {
        if (!EnsurePages(kv_[0]->PagesNeeded(ms.internal_id, need) + 1))
          throw std::runtime_error("not enough KV memory to receive the request");
        plan = kv_[0]->BeginForward({ms.internal_id}, {static_cast<int32_t>(need)});
        if (!plan.page_copies.empty()) backend_->ApplyPageCopies(0, plan.page_copies);
      }
      rs->disagg_reserved_end = end;
      rs->disagg_matched = matched;
      e.status = EntryStatus::kAlive;  // holds a sequence; not schedulable until start-generation
      ms.inputs.clear();
      json::Array slots;
      for (int32_t sl : plan.slots) slots.push_back(Value(static_cast<int64_t>(sl)));
      Object meta;
      meta["slots"] = Value(std::move(slots));
      meta["begin"] = matched;
      meta["end"] = end;
      Object disagg;
      disagg["kv_append_metadata"] = Value(Value(std::move(meta)).dump());
      disagg["prefix_matched_length"] = matched;
      RequestStreamOutput out;
      out.request_id = req.id;
      out.group_delta_token_ids.resize(1);
      out.group_delta_logprob_json_strs.resize(1);
      out.group_finish_reason = {"stop"};
      out.group_extra_prefix_string = {""};
      Value usage = rs->metrics.AsUsageJSON(true);
      usage.as_object()["extra"].as_object()["disagg"] = Value(Value(std::move(disagg)).dump());
      out.request_final_usage_json_str = usage.dump();
      Emit({std::move(out)});
    } catch (...) {
      for (auto& e : rs->entries) ReleaseEntry(e, /*recycle=*/false);
      states_.erase(req.id);
      throw;
    }
  }

  // Decode side, step 3: the KV of [0, begin) has arrived; prefill the rest locally and decode.
  // Returns false when no reservation exists for this id (the request then runs as a normal one).
  bool TakeOverReservedRequest(RequestState* incoming) {
    auto it = states_.find(incoming->request.id);
    if (it == states_.end() || it->second->disagg_reserved_end < 0) return false;
    RequestState* rs = it->second.get();
    const DisaggConfig& dc = incoming->request.cfg.debug_config.disagg_config;
    const int64_t begin = dc.kv_window_begin.value_or(rs->disagg_reserved_end);
    if (begin != rs->disagg_reserved_end)
      throw std::runtime_error("start-generation position does not match the reserved KV range");
    std::vector<int32_t> tokens = AllTokens(incoming->request);
    if (static_cast<int64_t>(tokens.size()) <= begin) throw std::runtime_error("nothing left to prefill");
    rs->request.cfg = incoming->request.cfg;
    rs->request.cfg.debug_config.disagg_config = DisaggConfig();
    rs->request.inputs = incoming->request.inputs;
    rs->request.prompt_tokens = static_cast<int64_t>(tokens.size());
    rs->metrics = RequestMetrics();
    rs->metrics.prompt_tokens = rs->request.prompt_tokens;
    rs->metrics.add_time = NowSeconds();
    RequestStateEntry& e = rs->entries[0];
    ModelState& ms = e.mstates[0];
    e.stop_handler = std::make_unique<StopStrHandler>(rs->request.cfg.stop_strs, tok_);
    if (rs->request.cfg.seed >= 0) e.rng.seed(static_cast<uint64_t>(rs->request.cfg.seed));
    // received tokens become part of the cached prefix of this sequence
    if (prefix_cache_.HasSequence(ms.internal_id) && begin > rs->disagg_matched) {
      std::vector<int32_t> got(tokens.begin() + rs->disagg_matched, tokens.begin() + begin);
      prefix_cache_.ExtendSequence(ms.internal_id, got);
      prefix_cache_.CommitSequenceExtention();
    }
    ms.prefilled_tokens.assign(tokens.begin(), tokens.begin() + begin);
    ms.num_prefilled_tokens = begin;
    ms.inputs.clear();
    InputItem rest;
    rest.tokens.assign(tokens.begin() + begin, tokens.end());
    ms.inputs.push_back(std::move(rest));
    rs->disagg_reserved_end = -1;
    rs->num_unfinished = 1;
    running_.push_back(rs);  // it already owns a KV sequence: a running request with inputs left
    return true;
  }

  // Prefill side: after [0, end) is computed, copy the KV of [begin, end) to the receiver.
  void SendKVOfFinishedEntry(RequestState* rs, RequestStateEntry& e) {
    const DisaggConfig& dc = rs->request.cfg.debug_config.disagg_config;
    const int64_t id = e.mstates[0].internal_id;
    if (id < 0 || !kv_[0]->Has(id)) return;
    const int64_t end = rs->request.prompt_tokens;
    const int64_t begin = std::max<int64_t>(0, std::min<int64_t>(dc.kv_window_begin.value_or(0), end));
    if (begin >= end) return;
    std::vector<int32_t> pages = kv_[0]->SequencePages(id);
    const int64_t page = cfg_.kv_cache_page_size;
    std::vector<int32_t> slots;
    for (int64_t pos = begin; pos < end; ++pos)
      slots.push_back(static_cast<int32_t>(pages[pos / page] * page + pos % page));
    backend_->SendKV(0, slots, dc.kv_append_metadata);
  }

  void AbortRequest(const std::string& request_id) override {
    auto it = states_.find(request_id);
    if (it == states_.end()) return;
    RequestState* rs = it->second.get();
    ForgetInflight(rs);
    Trace(request_id, "abort");
    for (auto& e : rs->entries) ReleaseEntry(e, /*recycle=*/false);
    RemoveFromQueues(rs);
    states_.erase(it);
  }

  // A decode step whose result was never read is read and thrown away (its requests are gone).
  void DiscardInflightDecode() {
    if (inflight_.active && backend_) {
      try {
        backend_->WaitSample(0);
      } catch (...) {  // the step itself may be what failed
      }
    }
    inflight_ = InflightDecode();
  }

  void AbortAllRequests() override {
    DiscardInflightDecode();
    std::vector<std::string> ids;
    for (auto& kv : states_) ids.push_back(kv.first);
    for (auto& id : ids) AbortRequest(id);
  }

  void Reset() override {
    AbortAllRequests();
    running_.clear();
    waiting_.clear();
    states_.clear();
    prefix_cache_.Reset();
    for (auto& kv : kv_) kv->Clear();
    ids_.Reset();
    if (spec_) draft_slots_.Resize(static_cast<int>(cfg_.max_num_sequence) * DraftSlotsPerSequence());
    metrics_.Reset();
    if (backend_) backend_->Reset();
  }

  void Step() override {
    touched_.clear();
    // A decode step whose tokens have not been read yet is finished first whenever the next thing to do
    // is not another plain decode step (new requests to prefill, forced tokens, ...).
    if (inflight_.active && !PipelinedDecodePossible()) {
      FinishInflightDecode();
      const double t0 = NowSeconds();
      PostProcess();
      t_post_ += NowSeconds() - t0;
      return;
    }
    StepJumpForward();
    bool did = inflight_.active ? false : StepPrefill();
    if (!did) {
      if (spec_) did = StepSpecDecode();
      else if (PipelinedDecodePossible()) did = StepDecodePipelined();
      else did = StepDecode();
    }
    if (did) {
      const double t0 = NowSeconds();
      PostProcess();
      t_post_ += NowSeconds() - t0;
    }
  }

 private:
  // ---------------------------------------------------------------- helpers
  int MaxDraftLength() const { return cfg_.spec_draft_length > 0 ? cfg_.spec_draft_length : 4; }
  // Distribution slots one sequence can hold at once: a chain needs one per draft token; a tree one per
  // node that gets children (1 + w + ... + w^(k-1)).
  int DraftSlotsPerSequence() const {
    const int k = MaxDraftLength();
    int rows = 1, level = 1;
    for (int d = 1; d < k; ++d) {
      level *= std::max(1, cfg_.spec_tree_width);
      rows += level;
    }
    return std::max(2 * (k + 1), rows + 1);
  }

  void Trace(const std::string& id, const std::string& ev) {
    if (trace_) trace_->AddEvent(id, ev);
  }
  void TraceBatch(const std::vector<EntryRef>& batch, const std::string& ev) {
    if (!trace_) return;
    std::vector<std::string> ids;
    for (auto& r : batch) ids.push_back(r.rs->request.id);
    trace_->AddEvent(ids, ev);
  }
  void Emit(std::vector<RequestStreamOutput> outs) {
    if (callback_ && !outs.empty()) callback_(std::move(outs));
  }
  void Touch(RequestState* rs) {
    if (std::find(touched_.begin(), touched_.end(), rs) == touched_.end()) touched_.push_back(rs);
  }
  void RemoveFromQueues(RequestState* rs) {
    running_.erase(std::remove(running_.begin(), running_.end(), rs), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), rs), waiting_.end());
  }

  void OnPrefixCacheRemove(int64_t id) {
    for (auto& kv : kv_)
      if (kv->Has(id)) kv->RemoveSequence(id);
    ids_.Recycle(id);
  }

  // Frees everything an entry holds. recycle == true hands the sequence to the prefix cache.
  void ReleaseEntry(RequestStateEntry& e, bool recycle) {
    if (e.kv_released) return;
    e.kv_released = true;
    if (e.grammar_handle >= 0 && grammar_) {
      grammar_->Release(e.grammar_handle);
      e.grammar_handle = -1;
    }
    for (auto& ms : e.mstates) {
      for (int s : ms.draft_slots) draft_slots_.Free(s);
      ms.draft_slots.clear();
      ms.draft_tokens.clear();
      ms.draft_parents.clear();
      for (auto& in : ms.inputs)
        if (in.kind == 1 && backend_) backend_->ReleaseEmbedding(in.embed_handle);
    }
    const int64_t id = e.mstates[0].internal_id;
    if (id < 0) return;
    for (auto& ms : e.mstates) ms.internal_id = -1;
    if (prefix_cache_.HasSequence(id)) {
      if (recycle) {
        // the cache indexes exactly the tokens it was told about: drop any KV beyond them
        const int64_t keep = prefix_cache_.SequenceLength(id);
        for (auto& kv : kv_)
          if (kv->Has(id) && kv->SequenceLength(id) > keep) kv->PopN(id, kv->SequenceLength(id) - keep);
      }
      prefix_cache_.RecycleSequence(id, recycle);  // may call OnPrefixCacheRemove
    } else {
      OnPrefixCacheRemove(id);
    }
  }

  int64_t NumActiveSequences() const {
    int64_t n = 0;
    for (RequestState* rs : running_)
      for (auto& e : rs->entries)
        if (!e.kv_released && e.mstates[0].internal_id >= 0) ++n;
    return n;
  }

  std::vector<EntryRef> ReadyToDecode() {
    std::vector<EntryRef> out;
    for (RequestState* rs : running_)
      for (int i = 0; i < static_cast<int>(rs->entries.size()); ++i) {
        RequestStateEntry& e = rs->entries[i];
        if (e.status == EntryStatus::kAlive && e.mstates[0].inputs.empty() && !e.committed_tokens.empty())
          out.push_back({rs, i});
      }
    return out;
  }

  bool IsStopToken(const Request& req, int32_t token) const {
    for (int t : req.cfg.stop_token_ids)
      if (t == token) return true;
    if (!req.cfg.debug_config.ignore_eos)
      for (int32_t t : models_[0].eos_token_ids)
        if (t == token) return true;
    return false;
  }

  void CommitToken(EntryRef r, const SampleResult& s) {
    RequestStateEntry& e = r.e();
    e.committed_tokens.push_back(s);
    ++e.appeared_token_ids[s.token];
    ++r.rs->metrics.completion_tokens;
    if (e.grammar_handle >= 0 && grammar_ && !IsStopToken(r.rs->request, s.token))
      grammar_->AcceptToken(e.grammar_handle, s.token);
    Touch(r.rs);
  }

  // Appends the sampling parameters of one row. `path`: draft tokens that precede this row's position beyond the
  // committed ones (the row of a draft-tree node, or of a draft round, follows its ancestors): the penalties
  // count them and the grammar mask is the one of the state after them, as if they had been committed.
  void AddSampleRow(SampleParams* sp, EntryRef r, int32_t logit_token_index,
                    const std::vector<int32_t>* path = nullptr) {
    RequestStateEntry& e = r.e();
    const GenerationConfig& g = r.rs->request.cfg;
    if (path && path->empty()) path = nullptr;
    if (path) {
      const bool pen = g.frequency_penalty != 0 || g.presence_penalty != 0 || g.repetition_penalty != 1.0;
      const bool gram = e.grammar_handle >= 0 && grammar_;
      if (!pen && !gram) path = nullptr;
    }
    int accepted = 0;
    bool dead = false;  // the path leaves the grammar: the node can never be accepted, any mask will do
    if (path) {
      for (int32_t t : *path) ++e.appeared_token_ids[t];
      if (e.grammar_handle >= 0 && grammar_)
        for (int32_t t : *path) {
          if (IsStopToken(r.rs->request, t) || !grammar_->AcceptToken(e.grammar_handle, t)) {
            dead = true;
            break;
          }
          ++accepted;
        }
    }
    AddSampleRowNow(sp, r, logit_token_index, dead);
    if (path) {
      if (accepted > 0) grammar_->Rollback(e.grammar_handle, accepted);
      for (int32_t t : *path) {
        auto it = e.appeared_token_ids.find(t);
        if (it != e.appeared_token_ids.end() && --it->second <= 0) e.appeared_token_ids.erase(it);
      }
    }
  }

  void AddSampleRowNow(SampleParams* sp, EntryRef r, int32_t logit_token_index, bool skip_grammar) {
    RequestStateEntry& e = r.e();
    const GenerationConfig& g = r.rs->request.cfg;
    const int row = static_cast<int>(sp->logit_token_index.size());
    sp->logit_token_index.push_back(logit_token_index);
    sp->temperature.push_back(static_cast<float>(g.temperature));
    sp->top_p.push_back(static_cast<float>(g.top_p));
    sp->top_k.push_back(g.top_k);
    sp->uniform.push_back(static_cast<float>(e.NextUniform()));
    const bool has_pen = g.frequency_penalty != 0 || g.presence_penalty != 0 || g.repetition_penalty != 1.0;
    sp->penalties.push_back(static_cast<float>(g.presence_penalty));
    sp->penalties.push_back(static_cast<float>(g.frequency_penalty));
    sp->penalties.push_back(static_cast<float>(g.repetition_penalty));
    if (has_pen)
      for (auto& kv : e.appeared_token_ids) {
        sp->pen_row.push_back(row);
        sp->pen_token.push_back(kv.first);
        sp->pen_count.push_back(kv.second);
      }
    for (auto& b : g.logit_bias) {
      sp->bias_row.push_back(row);
      sp->bias_token.push_back(b.first);
      sp->bias_value.push_back(b.second);
    }
    if (e.grammar_handle >= 0 && grammar_ && !skip_grammar) {
      std::vector<int32_t> bits = grammar_->NextTokenBitmask(e.grammar_handle);
      sp->mask_rows.push_back(row);
      sp->mask_bits.insert(sp->mask_bits.end(), bits.begin(), bits.end());
    }
    if (g.logprobs) sp->num_top_logprobs = std::max(sp->num_top_logprobs, g.top_logprobs);
  }

  SampleResult RowResult(const SampleOutput& out, int row, int num_top, const GenerationConfig& g) {
    SampleResult s;
    s.token = out.tokens[row];
    s.prob = row < static_cast<int>(out.probs.size()) ? out.probs[row] : 1.f;
    if (g.logprobs && num_top > 0)
      for (int k = 0; k < g.top_logprobs && k < num_top; ++k)
        s.top.emplace_back(out.top_tokens[row * num_top + k], out.top_probs[row * num_top + k]);
    return s;
  }

  // Makes room for `pages` KV pages in model 0, evicting recycled prefixes first.
  bool EnsurePages(int64_t pages) {
    while (kv_[0]->NumAvailablePages() < pages) {
      if (!prefix_cache_.TryFreeMemory()) return false;
    }
    return true;
  }

  // ---------------------------------------------------------------- preemption
  void PreemptLast() {
    // last alive entry of the last running request
    for (auto rit = running_.rbegin(); rit != running_.rend(); ++rit) {
      RequestState* rs = *rit;
      for (int i = static_cast<int>(rs->entries.size()) - 1; i >= 0; --i) {
        RequestStateEntry& e = rs->entries[i];
        if (e.status != EntryStatus::kAlive || e.mstates[0].internal_id < 0) continue;
        Trace(rs->request.id, "preempt");
        ++num_preemptions_;
        const int64_t id = e.mstates[0].internal_id;
        // drop the KV now (non-lazy): memory is what we are short of
        if (prefix_cache_.HasSequence(id)) prefix_cache_.RecycleSequence(id, /*lazy=*/false);
        else OnPrefixCacheRemove(id);
        for (auto& ms : e.mstates) {
          for (int s : ms.draft_slots) draft_slots_.Free(s);
          ms = ModelState();
          for (auto& in : rs->request.inputs) ms.inputs.push_back(in);
          if (!e.committed_tokens.empty()) {
            InputItem it;
            for (auto& c : e.committed_tokens) it.tokens.push_back(c.token);
            ms.inputs.push_back(std::move(it));
          }
          // those tokens reach the prefix cache again as prefilled inputs
          ms.cached_committed_tokens = static_cast<int64_t>(e.committed_tokens.size());
        }
        e.status = EntryStatus::kPending;
        e.parent_idx = -1;  // re-prefilled as a self-contained sequence
        // if nothing of this request still runs, move it to the front of the waiting queue
        bool any_alive = false;
        for (auto& o : rs->entries) any_alive |= (o.status == EntryStatus::kAlive);
        if (!any_alive) {
          running_.erase(std::remove(running_.begin(), running_.end(), rs), running_.end());
          waiting_.insert(waiting_.begin(), rs);
        }
        return;
      }
    }
    throw std::runtime_error("Engine: nothing left to preempt");
  }

  // ---------------------------------------------------------------- prefill
  struct PrefillItem {
    EntryRef ref;
    int64_t take;       // tokens of this step
    bool completes;     // inputs exhausted after this step
    bool is_decode;     // hybrid: a running sequence contributing its single next token
  };

  // First scheduling of an entry: allocate / fork / reuse its KV sequence.
  void MatchPrefixAndCreateSequence(EntryRef r) {
    RequestStateEntry& e = r.e();
    ModelState& ms = e.mstates[0];
    std::vector<int32_t> tokens;
    bool all_tokens = true;
    for (auto& in : ms.inputs) {
      if (in.kind != 0) { all_tokens = false; break; }
      tokens.insert(tokens.end(), in.tokens.begin(), in.tokens.end());
    }
    int64_t id = ids_.Get();
    int64_t offset = 0;
    int64_t draft_offset = 0;
    if (all_tokens && prefix_cache_.enabled()) {
      PrefixMatch m = prefix_cache_.InsertSequence(id, tokens, static_cast<int>(cfg_.sliding_window_size),
                                                   static_cast<int>(std::max<int64_t>(0, cfg_.attention_sink_size)));
      if (m.reused_seq_id >= 0) {
        ids_.Recycle(id);
        id = m.reused_seq_id;
        offset = m.prefilled_offset;
        if (kv_[0]->SequenceLength(id) > offset) kv_[0]->PopN(id, kv_[0]->SequenceLength(id) - offset);
        for (size_t d = 1; d < kv_.size(); ++d) {
          if (!kv_[d]->Has(id)) kv_[d]->AddSequence(id);
          const int64_t dl = kv_[d]->SequenceLength(id);
          if (dl > offset) kv_[d]->PopN(id, dl - offset);
          draft_offset = std::min(dl, offset);
        }
      } else if (m.forked_seq_id >= 0) {
        // the fork may need a page for the copy-on-write of the last partial page
        EnsurePages(1);
        kv_[0]->ForkSequence(m.forked_seq_id, id, m.prefilled_offset);
        offset = m.prefilled_offset;
        for (size_t d = 1; d < kv_.size(); ++d) {
          if (kv_[d]->Has(m.forked_seq_id) && kv_[d]->NumAvailablePages() > 0) {
            draft_offset = std::min(kv_[d]->SequenceLength(m.forked_seq_id), offset);
            kv_[d]->ForkSequence(m.forked_seq_id, id, draft_offset);
          } else {
            kv_[d]->AddSequence(id);
          }
        }
      } else {
        for (auto& kv : kv_) kv->AddSequence(id);
      }
      if (r.rs->request.cfg.debug_config.pinned_system_prompt) prefix_cache_.PinSequence(id);
    } else {
      for (auto& kv : kv_) kv->AddSequence(id);
    }
    // every sequence is windowed, parents of parallel samples too: the window is part of what a token sees
    // (a mask), and pages that fall out of it are reference-counted, so sharing them with forks is safe;
    // forked children inherit the window (KVManager::ForkSequence)
    if (cfg_.sliding_window_size > 0)
      for (auto& kv : kv_)
        kv->EnableSlidingWindow(id, static_cast<int32_t>(cfg_.sliding_window_size),
                                static_cast<int32_t>(std::max<int64_t>(0, cfg_.attention_sink_size)));
    for (auto& s : e.mstates) s.internal_id = id;
    auto drop_prefix = [](ModelState& st, int64_t n) {
      st.num_prefilled_tokens = n;
      int64_t left = n;
      while (left > 0 && !st.inputs.empty()) {
        InputItem& in = st.inputs.front();
        if (static_cast<int64_t>(in.tokens.size()) <= left) {
          left -= static_cast<int64_t>(in.tokens.size());
          st.inputs.pop_front();
        } else {
          in.tokens.erase(in.tokens.begin(), in.tokens.begin() + left);
          left = 0;
        }
      }
    };
    if (offset > 0) {
      // drop the matched prefix from the pending inputs
      ms.prefilled_tokens.assign(tokens.begin(), tokens.begin() + offset);
      drop_prefix(ms, offset);
    }
    for (size_t d = 1; d < e.mstates.size(); ++d)
      if (draft_offset > 0) drop_prefix(e.mstates[d], draft_offset);
  }

  bool StepPrefill() {
    const double t0 = NowSeconds();
    // candidates in priority order: running requests with leftover inputs, then waiting requests
    std::vector<EntryRef> cands;
    auto collect = [&](RequestState* rs) {
      for (int i = 0; i < static_cast<int>(rs->entries.size()); ++i) {
        RequestStateEntry& e = rs->entries[i];
        if (e.status == EntryStatus::kFinished) continue;
        if (!e.mstates[0].inputs.empty()) cands.push_back({rs, i});
      }
    };
    for (RequestState* rs : running_) collect(rs);
    for (RequestState* rs : waiting_) collect(rs);
    if (cands.empty()) return false;

    std::vector<EntryRef> decode_ready = ReadyToDecode();
    int64_t budget = cfg_.prefill_chunk_size;
    int64_t active = NumActiveSequences();
    int64_t pages_reserved = 0;
    int64_t total_new = 0;
    std::vector<PrefillItem> items;
    const int64_t page = cfg_.kv_cache_page_size;
    for (EntryRef r : cands) {
      if (budget <= 0) break;
      RequestStateEntry& e = r.e();
      ModelState& ms = e.mstates[0];
      const bool is_new = ms.internal_id < 0;
      if (is_new) {
        const int64_t seqs_needed = 1 + static_cast<int64_t>(e.child_indices.size());
        if (active + seqs_needed > cfg_.max_num_sequence) break;
        // memory admission is evaluated on the unmatched length (a prefix hit only helps)
        int64_t input_len = 0;
        for (auto& in : ms.inputs) input_len += in.Length();
        const int64_t first_take = std::min(input_len, budget);
        const int64_t need = (first_take + page - 1) / page + 1 + seqs_needed;
        if (!EnsurePages(pages_reserved + need)) break;
        if (kv_[0]->TotalSequenceLength() + total_new + first_take + 8 * (active + seqs_needed) >
            cfg_.max_total_sequence_length) {
          // try to shed cached prefixes, then give up for this step
          bool freed = false;
          while (prefix_cache_.TryFreeMemory()) {
            freed = true;
            if (kv_[0]->TotalSequenceLength() + total_new + first_take + 8 * (active + seqs_needed) <=
                cfg_.max_total_sequence_length)
              break;
          }
          if (!freed || kv_[0]->TotalSequenceLength() + total_new + first_take + 8 * (active + seqs_needed) >
                            cfg_.max_total_sequence_length)
            break;
        }
        MatchPrefixAndCreateSequence(r);
        active += seqs_needed;
        if (std::find(running_.begin(), running_.end(), r.rs) == running_.end()) {
          waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r.rs), waiting_.end());
          running_.push_back(r.rs);
        }
        e.status = EntryStatus::kAlive;
      }
      int64_t input_len = 0;
      for (auto& in : ms.inputs) input_len += in.Length();
      if (input_len == 0) continue;  // fully matched by the prefix cache (cannot happen: last token kept)
      int64_t take = std::min(input_len, budget);
      // embeddings are never split
      if (take < input_len) {
        int64_t acc = 0;
        for (auto& in : ms.inputs) {
          if (acc + in.Length() <= take) { acc += in.Length(); continue; }
          if (in.kind == 1) take = acc;  // stop before this embedding item
          break;
        }
        if (take == 0) break;
      }
      const int64_t need = kv_[0]->PagesNeeded(ms.internal_id, take) + 1;
      if (!EnsurePages(pages_reserved + need)) {
        if (items.empty() && decode_ready.empty()) {
          // nothing else can make progress: shed the newest running sequence
          if (NumActiveSequences() > 1) { PreemptLast(); return true; }
        }
        break;
      }
      pages_reserved += need;
      total_new += take;
      budget -= take;
      items.push_back({r, take, take == input_len, false});
    }
    if (items.empty()) return false;
    if (cfg_.prefill_mode == PrefillMode::kHybrid) {
      for (EntryRef r : decode_ready) {
        if (budget <= 0) break;
        const int64_t need = kv_[0]->PagesNeeded(r.e().mstates[0].internal_id, 1);
        if (!EnsurePages(pages_reserved + need)) break;
        pages_reserved += need;
        budget -= 1;
        r.rs->metrics.decode_tokens += 1;
        items.push_back({r, 1, true, true});
      }
    }
    std::vector<EntryRef> batch;
    for (auto& it : items) batch.push_back(it.ref);
    TraceBatch(batch, "start prefill");

    // ---- assemble the model call
    std::vector<int64_t> seq_ids;
    std::vector<int32_t> lens, token_ids;
    std::vector<int64_t> embed_handles;
    SampleParams sp;
    struct RowOwner { EntryRef ref; int child; };
    std::vector<RowOwner> owners;
    int32_t tok_off = 0;
    for (auto& it : items) {
      RequestStateEntry& e = it.ref.e();
      ModelState& ms = e.mstates[0];
      seq_ids.push_back(ms.internal_id);
      lens.push_back(static_cast<int32_t>(it.take));
      if (it.is_decode) {
        token_ids.push_back(e.committed_tokens.back().token);
        embed_handles.push_back(-1);
      } else {
        int64_t left = it.take;
        std::vector<int32_t> fed;
        while (left > 0) {
          InputItem& in = ms.inputs.front();
          if (in.kind == 1) {
            for (int32_t k = 0; k < in.embed_len; ++k) {
              token_ids.push_back(k);  // row inside the embedding
              embed_handles.push_back(in.embed_handle);
            }
            left -= in.embed_len;
            ms.inputs.pop_front();
            continue;
          }
          const int64_t n = std::min<int64_t>(left, static_cast<int64_t>(in.tokens.size()));
          token_ids.insert(token_ids.end(), in.tokens.begin(), in.tokens.begin() + n);
          embed_handles.insert(embed_handles.end(), n, -1);
          fed.insert(fed.end(), in.tokens.begin(), in.tokens.begin() + n);
          if (n == static_cast<int64_t>(in.tokens.size())) ms.inputs.pop_front();
          else in.tokens.erase(in.tokens.begin(), in.tokens.begin() + n);
          left -= n;
        }
        ms.num_prefilled_tokens += it.take;
        ms.prefilled_tokens.insert(ms.prefilled_tokens.end(), fed.begin(), fed.end());
        const int64_t forced = std::min<int64_t>(it.take, ms.jump_forward_inputs);
        ms.jump_forward_inputs -= forced;
        it.ref.rs->metrics.prefill_tokens += it.take - forced;
        if (prefix_cache_.HasSequence(ms.internal_id)) prefix_cache_.ExtendSequence(ms.internal_id, fed);
      }
      if (it.completes) {
        const int32_t last = tok_off + static_cast<int32_t>(it.take) - 1;
        if (!it.is_decode && !e.child_indices.empty()) {
          for (int c : e.child_indices) {
            AddSampleRow(&sp, {it.ref.rs, c}, last);
            owners.push_back({it.ref, c});
          }
        } else {
          AddSampleRow(&sp, it.ref, last);
          owners.push_back({it.ref, -1});
        }
      }
      tok_off += static_cast<int32_t>(it.take);
    }
    ForwardPlan plan = kv_[0]->BeginForward(seq_ids, lens);
    SampleOutput out = backend_->ForwardSample(0, plan, token_ids, embed_handles, sp);
    prefix_cache_.CommitSequenceExtention();
    if (spec_) PrefillDraftModel(items);

    // ---- commit
    const double now = NowSeconds();
    for (size_t row = 0; row < owners.size(); ++row) {
      EntryRef parent = owners[row].ref;
      const GenerationConfig& g = parent.rs->request.cfg;
      SampleResult s = RowResult(out, static_cast<int>(row), sp.num_top_logprobs, g);
      if (owners[row].child >= 0) {
        EntryRef child{parent.rs, owners[row].child};
        RequestStateEntry& ce = child.e();
        const int64_t cid = ids_.Get();
        EnsurePages(1);
        for (size_t m = 0; m < kv_.size(); ++m)
          if (kv_[m]->Has(parent.e().mstates[m].internal_id))
            kv_[m]->ForkSequence(parent.e().mstates[m].internal_id, cid, -1);
        for (auto& ms : ce.mstates) ms.internal_id = cid;
        ce.mstates[0].prefilled_tokens = parent.e().mstates[0].prefilled_tokens;
        ce.status = EntryStatus::kAlive;
        CommitToken(child, s);
      } else {
        CommitToken(parent, s);
      }
      if (!parent.rs->prefill_done) {
        parent.rs->prefill_done = true;
        parent.rs->metrics.prefill_end_time = now;
      }
    }
    // a parent whose children took over stays only as the holder of the shared prompt KV
    for (auto& it : items)
      if (it.completes && !it.is_decode && !it.ref.e().child_indices.empty())
        it.ref.e().status = EntryStatus::kFinished;
    for (auto& it : items) Touch(it.ref.rs);
    TraceBatch(batch, "finish prefill");
    ++num_prefill_steps_;
    metrics_.engine_prefill_time_sum += NowSeconds() - t0;
    return true;
  }

  // ---------------------------------------------------------------- decode
  // Shrinks `ready` (preempting from the back) until one token per sequence fits in memory.
  bool FitDecodeBatch(std::vector<EntryRef>* ready, int64_t tokens_per_seq) {
    while (!ready->empty()) {
      int64_t need = 0;
      for (auto& r : *ready) need += kv_[0]->PagesNeeded(r.e().mstates[0].internal_id, tokens_per_seq);
      if (EnsurePages(need)) return true;
      if (ready->size() == 1 && NumActiveSequences() <= 1)
        throw std::runtime_error("Engine: KV cache too small for a single sequence");
      PreemptLast();
      *ready = ReadyToDecode();
    }
    return false;
  }

  // ---------------------------------------------------------------- pipelined decode
  // Plain decode steps overlap the host with the device: step n + 1 is planned and queued while step n
  // still runs, its input tokens being the tokens step n samples, which stay on the device; step n's
  // tokens reach the host (and the request's stream) while step n + 1 runs. A sequence that turns out
  // to have ended with step n (stop token, stop string) has then been scheduled once too often: the
  // extra token is dropped and its KV entry goes away with the sequence. Ends by length are known in
  // advance and are not scheduled again. Anything that needs the newest token on the host before the
  // next step can be planned (grammar masks, repetition penalties, speculative decoding, forced
  // tokens, a second model) takes the ordinary synchronous path.
  struct InflightRow {
    RequestState* rs;  // null once the request was aborted
    int idx;
  };
  struct InflightDecode {
    bool active = false;
    std::vector<InflightRow> rows;
    int num_top_logprobs = 0;
    double t_launch = 0;
  };

  // The request object goes away: whatever the unread step still samples for it is dropped on arrival.
  void ForgetInflight(const RequestState* rs) {
    for (auto& row : inflight_.rows)
      if (row.rs == rs) row.rs = nullptr;
  }

  bool EntryNeedsHostToken(const RequestState& rs, const RequestStateEntry& e) const {
    const GenerationConfig& g = rs.request.cfg;
    return e.grammar_handle >= 0 || g.frequency_penalty != 0 || g.presence_penalty != 0 ||
           g.repetition_penalty != 1.0 || rs.request.cfg.debug_config.disagg_config.kind != DisaggRequestKind::kNone;
  }

  bool PipelinedDecodePossible() const {
    if (!pipelined_decode_ || pipelined_pause_ || spec_ || kv_.size() != 1 || !waiting_.empty() || running_.empty())
      return false;
    for (const RequestState* rs : running_) {
      if (rs->disagg_reserved_end >= 0) return false;
      for (const RequestStateEntry& e : rs->entries) {
        if (e.status == EntryStatus::kPending) return false;
        if (e.status != EntryStatus::kAlive) continue;
        if (!e.mstates[0].inputs.empty() || EntryNeedsHostToken(*rs, e)) return false;
      }
    }
    return true;
  }

  // Tokens an entry may still be scheduled for, counting the one in flight.
  bool ReachesLengthLimit(const RequestState& rs, const RequestStateEntry& e) const {
    const int64_t produced = static_cast<int64_t>(e.committed_tokens.size()) + (e.inflight_row >= 0 ? 1 : 0);
    if (rs.request.cfg.max_tokens >= 0 && produced >= rs.request.cfg.max_tokens) return true;
    return rs.request.prompt_tokens + produced >= cfg_.max_single_sequence_length;
  }

  void FinishInflightDecode() {
    if (!inflight_.active) return;
    const double tb = NowSeconds();
    SampleOutput out = backend_->WaitSample(0);
    const double tc = NowSeconds();
    InflightDecode done = std::move(inflight_);
    inflight_ = InflightDecode();
    for (size_t i = 0; i < done.rows.size(); ++i) {
      RequestState* rs = done.rows[i].rs;
      if (rs == nullptr) {  // the request ended (or was aborted) with the step before: one token too many
        ++num_dropped_tokens_;
        continue;
      }
      RequestStateEntry& e = rs->entries[done.rows[i].idx];
      if (e.inflight_row == static_cast<int>(i)) e.inflight_row = -1;
      if (e.status != EntryStatus::kAlive) {  // ended with the step before: one token too many
        ++num_dropped_tokens_;
        continue;
      }
      rs->metrics.decode_tokens += 1;
      CommitToken({rs, done.rows[i].idx},
                  RowResult(out, static_cast<int>(i), done.num_top_logprobs, rs->request.cfg));
    }
    t_backend_ += tc - tb;
    t_commit_ += NowSeconds() - tc;
    ++num_decode_steps_;
    ++num_pipelined_steps_;
    const double dt = NowSeconds() - done.t_launch;
    metrics_.engine_decode_time_sum += dt;
    metrics_.UpdateDecodeTimeByBatchSize(static_cast<int>(done.rows.size()), dt);
  }

  bool StepDecodePipelined() {
    const double t0 = NowSeconds();
    std::vector<EntryRef> ready;
    for (RequestState* rs : running_)
      for (int i = 0; i < static_cast<int>(rs->entries.size()); ++i) {
        RequestStateEntry& e = rs->entries[i];
        if (e.status != EntryStatus::kAlive || !e.mstates[0].inputs.empty()) continue;
        if (e.committed_tokens.empty() && e.inflight_row < 0) continue;
        if (ReachesLengthLimit(*rs, e)) continue;  // its last token is in flight or waits for post-processing
        ready.push_back({rs, i});
      }
    if (static_cast<int64_t>(ready.size()) > cfg_.max_num_sequence) ready.resize(cfg_.max_num_sequence);
    bool launched = false;
    InflightDecode next;
    if (!ready.empty()) {
      int64_t need = 0;
      for (auto& r : ready) need += kv_[0]->PagesNeeded(r.e().mstates[0].internal_id, 1);
      if (!EnsurePages(need)) {
        // out of pages: preemption works on settled state, so settle first and let the ordinary path decide
        FinishInflightDecode();
        pipelined_pause_ = true;
        return true;
      }
      TraceBatch(ready, "start decode");
      std::vector<int64_t> seq_ids;
      std::vector<int32_t> lens(ready.size(), 1), token_ids, token_src;
      SampleParams sp;
      for (size_t i = 0; i < ready.size(); ++i) {
        RequestStateEntry& e = ready[i].e();
        seq_ids.push_back(e.mstates[0].internal_id);
        token_src.push_back(e.inflight_row);
        token_ids.push_back(e.inflight_row >= 0 ? 0 : e.committed_tokens.back().token);
        AddSampleRow(&sp, ready[i], static_cast<int32_t>(i));
      }
      const double ta = NowSeconds();
      ForwardPlan plan = kv_[0]->BeginForward(seq_ids, lens);
      const double tb = NowSeconds();
      launched = backend_->LaunchSample(0, plan, token_ids, token_src, sp);
      t_assemble_ += ta - t0;
      t_plan_ += tb - ta;
      t_backend_ += NowSeconds() - tb;
      if (!launched) {
        // the backend cannot defer this step: undo the plan, settle, and stay on the ordinary path
        for (int64_t id : seq_ids) kv_[0]->PopN(id, 1);
        kv_[0]->RequeuePlanSideEffects(plan);  // copy-on-write page copies and forks ride on the next plan
        FinishInflightDecode();
        pipelined_decode_ = false;
        return true;
      }
      next.active = true;
      next.num_top_logprobs = sp.num_top_logprobs;
      next.t_launch = t0;
      for (size_t i = 0; i < ready.size(); ++i) next.rows.push_back({ready[i].rs, ready[i].idx});
    }
    if (!launched && !inflight_.active) return false;
    // the step before this one: its tokens reach the host while the new step runs
    FinishInflightDecode();
    if (launched) {
      for (size_t i = 0; i < next.rows.size(); ++i) next.rows[i].rs->entries[next.rows[i].idx].inflight_row = static_cast<int>(i);
      inflight_ = std::move(next);
    }
    return true;
  }

  bool StepDecode() {
    const double t0 = NowSeconds();
    pipelined_pause_ = false;
    std::vector<EntryRef> ready = ReadyToDecode();
    if (ready.empty()) return false;
    if (!FitDecodeBatch(&ready, 1)) return false;
    if (static_cast<int64_t>(ready.size()) > cfg_.max_num_sequence) ready.resize(cfg_.max_num_sequence);
    TraceBatch(ready, "start decode");
    std::vector<int64_t> seq_ids;
    std::vector<int32_t> lens(ready.size(), 1), token_ids;
    std::vector<int64_t> embed_handles(ready.size(), -1);
    SampleParams sp;
    for (size_t i = 0; i < ready.size(); ++i) {
      RequestStateEntry& e = ready[i].e();
      seq_ids.push_back(e.mstates[0].internal_id);
      token_ids.push_back(e.committed_tokens.back().token);
      AddSampleRow(&sp, ready[i], static_cast<int32_t>(i));
    }
    const double ta = NowSeconds();
    ForwardPlan plan = kv_[0]->BeginForward(seq_ids, lens);
    const double tb = NowSeconds();
    SampleOutput out = backend_->ForwardSample(0, plan, token_ids, embed_handles, sp);
    const double tc = NowSeconds();
    for (size_t i = 0; i < ready.size(); ++i) {
      ready[i].rs->metrics.decode_tokens += 1;
      CommitToken(ready[i], RowResult(out, static_cast<int>(i), sp.num_top_logprobs, ready[i].rs->request.cfg));
    }
    t_assemble_ += ta - t0;
    t_plan_ += tb - ta;
    t_backend_ += tc - tb;
    t_commit_ += NowSeconds() - tc;
    TraceBatch(ready, "finish decode");
    ++num_decode_steps_;
    const double dt = NowSeconds() - t0;
    metrics_.engine_decode_time_sum += dt;
    metrics_.UpdateDecodeTimeByBatchSize(static_cast<int>(ready.size()), dt);
    return true;
  }

  // ---------------------------------------------------------------- jump-forward decoding
  // When the grammar leaves only one way to continue (a JSON key, punctuation, ...), that text is
  // appended without running the model for each of its tokens (reference:
  // cpp/serve/engine_actions/batch_jumpforward.cc).  The tail of the output is re-tokenised together
  // with the forced text, because the natural tokenisation may merge across the seam: tokens that no
  // longer fit are rolled back (KV, grammar, prefix cache) and the new ones are committed.  The
  // committed-but-not-yet-computed tokens then become inputs of the sequence, so the next prefill
  // step computes their KV in one pass and samples the token that follows.
  static constexpr int kMaxRollbackTokens = 10;
  static constexpr int kJumpForwardPagesPerRequest = 10;

  void StepJumpForward() {
    if (!grammar_ || spec_ || kv_.size() > 1 || !tok_) return;
    std::vector<EntryRef> ready = ReadyToDecode();
    if (ready.empty()) return;
    bool any_grammar = false;
    for (auto& r : ready) any_grammar |= r.e().grammar_handle >= 0;
    if (!any_grammar) return;
    const double t0 = NowSeconds();
    // keep headroom for the forced text of every running request, as the reference does
    if (static_cast<int64_t>(ready.size()) * kJumpForwardPagesPerRequest > kv_[0]->NumAvailablePages() &&
        !EnsurePages(static_cast<int64_t>(ready.size()) * kJumpForwardPagesPerRequest))
      return;
    for (EntryRef r : ready) {
      RequestStateEntry& e = r.e();
      const GenerationConfig& g = r.rs->request.cfg;
      if (e.grammar_handle < 0 || g.logprobs ||
          g.debug_config.grammar_execution_mode != GrammarExecutionMode::kJumpForward)
        continue;
      if (grammar_->IsTerminated(e.grammar_handle)) continue;
      const std::string forced = grammar_->FindJumpForwardString(e.grammar_handle);
      if (forced.empty()) continue;
      JumpForward(r, forced);
    }
    metrics_.engine_jump_forward_time_sum += NowSeconds() - t0;
  }

  void JumpForward(EntryRef r, const std::string& forced) {
    RequestStateEntry& e = r.e();
    ModelState& ms = e.mstates[0];
    const int64_t n = static_cast<int64_t>(e.committed_tokens.size());
    // ---- re-tokenise the last few tokens together with the forced text
    const int64_t past_begin = std::max<int64_t>(0, n - kMaxRollbackTokens);
    std::vector<int32_t> past;
    std::string past_text;
    for (int64_t i = past_begin; i < n; ++i) {
      past.push_back(e.committed_tokens[i].token);
      past_text += tok_->TokenBytes(e.committed_tokens[i].token);
    }
    std::vector<int32_t> fresh = tok_->EncodeNoPrependSpace(past_text + forced);
    if (fresh.empty()) return;
    std::string delta_text = forced;
    // a last token that is a prefix of another token would likely be re-merged by the next decode
    // step; leave it (and its text) to the model
    const std::vector<bool>& prefix_mask = tok_->PrefixTokenMask();
    if (fresh.back() >= 0 && fresh.back() < static_cast<int32_t>(prefix_mask.size()) && prefix_mask[fresh.back()]) {
      const std::string& last = tok_->TokenBytes(fresh.back());
      if (last.size() >= forced.size()) return;
      delta_text.resize(delta_text.size() - last.size());
      fresh.pop_back();
    }
    size_t same = 0;
    while (same < past.size() && same < fresh.size() && past[same] == fresh[same]) ++same;
    const int64_t rollback = static_cast<int64_t>(past.size() - same);
    std::vector<int32_t> added(fresh.begin() + static_cast<std::ptrdiff_t>(same), fresh.end());
    if (rollback == 0 && added.empty()) return;

    // ---- stream output: text already handed out stays valid (the new tokens spell the same text plus
    // the forced part), so only the forced part is sent, as a string, and the new tokens are skipped
    if (rollback > n - e.next_callback_token_pos) {
      for (int64_t i = e.next_callback_token_pos; i < n; ++i)
        e.extra_prefix_string += tok_->TokenBytes(e.committed_tokens[i].token);
      e.extra_prefix_string += delta_text;
      e.next_callback_token_pos = n - rollback + static_cast<int64_t>(added.size());
    }
    // ---- roll back: grammar, token bookkeeping, prefix cache, KV
    if (rollback > 0) {
      grammar_->Rollback(e.grammar_handle, static_cast<int>(rollback));
      for (int64_t i = n - rollback; i < n; ++i) {
        auto it = e.appeared_token_ids.find(e.committed_tokens[i].token);
        if (it != e.appeared_token_ids.end() && --it->second <= 0) e.appeared_token_ids.erase(it);
      }
      e.committed_tokens.resize(n - rollback);
      r.rs->metrics.completion_tokens -= rollback;
      // the KV holds every committed token but the last one
      const int64_t kv_rollback = rollback - 1;
      if (kv_rollback > 0) {
        const int64_t cached = std::max<int64_t>(0, ms.cached_committed_tokens - (n - rollback));
        if (cached > 0 && prefix_cache_.HasSequence(ms.internal_id)) {
          prefix_cache_.RollBackSequence(ms.internal_id, cached);
          ms.cached_committed_tokens -= cached;
        }
        kv_[0]->PopN(ms.internal_id, kv_rollback);
      }
    }
    const int64_t in_kv = std::min<int64_t>(n - 1, n - rollback);  // committed tokens whose KV exists
    for (int32_t t : added) CommitToken(r, SampleResult{t, 1.f, {}});
    r.rs->metrics.jump_forward_tokens += std::max<int64_t>(0, static_cast<int64_t>(added.size()) - rollback);
    // ---- the tokens without KV become inputs; the next prefill step computes them and samples on
    InputItem item;
    for (int64_t i = in_kv; i < static_cast<int64_t>(e.committed_tokens.size()); ++i)
      item.tokens.push_back(e.committed_tokens[i].token);
    ms.jump_forward_inputs = static_cast<int64_t>(item.tokens.size());
    ms.inputs.push_back(std::move(item));
    // those tokens reach the prefix cache as prefilled inputs
    ms.cached_committed_tokens = static_cast<int64_t>(e.committed_tokens.size());
    Touch(r.rs);
  }

  // ---------------------------------------------------------------- speculative decoding
  int DraftLengthFor(int batch) const {
    if (cfg_.spec_draft_length > 0) return cfg_.spec_draft_length;
    // automatic mode: shorter drafts as the batch grows, plain decode for large batches
    if (batch < 10) return 4;
    if (batch < 20) return 3;
    if (batch < 30) return 2;
    return 0;
  }

  // Keeps the draft model's KV in step with the main model for the prompt part.
  void PrefillDraftModel(const std::vector<PrefillItem>& items) {
    std::vector<int64_t> seq_ids;
    std::vector<int32_t> lens, token_ids;
    std::vector<int64_t> embed_handles;
    for (auto& it : items) {
      RequestStateEntry& e = it.ref.e();
      ModelState& ms = e.mstates[1];
      if (it.is_decode) continue;  // the draft phase catches up on decode tokens by itself
      if (!kv_[1]->Has(ms.internal_id)) kv_[1]->AddSequence(ms.internal_id);
      // catch up to wherever the main model's prefill now stands
      int64_t left = e.mstates[0].num_prefilled_tokens - ms.num_prefilled_tokens;
      int64_t fed = 0;
      while (left > 0 && !ms.inputs.empty()) {
        InputItem& in = ms.inputs.front();
        if (in.kind == 1) {
          for (int32_t k = 0; k < in.embed_len; ++k) {
            token_ids.push_back(k);
            embed_handles.push_back(in.embed_handle);
          }
          left -= in.embed_len;
          fed += in.embed_len;
          ms.inputs.pop_front();
          continue;
        }
        const int64_t n = std::min<int64_t>(left, static_cast<int64_t>(in.tokens.size()));
        token_ids.insert(token_ids.end(), in.tokens.begin(), in.tokens.begin() + n);
        embed_handles.insert(embed_handles.end(), n, -1);
        if (n == static_cast<int64_t>(in.tokens.size())) ms.inputs.pop_front();
        else in.tokens.erase(in.tokens.begin(), in.tokens.begin() + n);
        left -= n;
        fed += n;
      }
      if (fed == 0) continue;
      ms.num_prefilled_tokens += fed;
      seq_ids.push_back(ms.internal_id);
      lens.push_back(static_cast<int32_t>(fed));
    }
    if (seq_ids.empty()) return;
    ForwardPlan plan = kv_[1]->BeginForward(seq_ids, lens);
    SampleParams none;
    backend_->ForwardSample(1, plan, token_ids, embed_handles, none);
  }

  // Draft tree (spec_tree_width > 1; reference: cpp/serve/engine_actions/batch_draft.cc:150-290): every
  // round gives each leaf `width` children, the most probable tokens of the draft model after that leaf;
  // the children share the slot that holds the leaf's distribution.  Round 0 feeds the tokens the draft
  // model has not seen and grows the first level; each later round feeds the whole tree built so far as
  // one chunk (the tree mask covers a chunk, so earlier levels are recomputed rather than left in the
  // KV, which keeps siblings invisible to each other) and grows its leaves.
  void DraftTree(const std::vector<EntryRef>& ready, int k, int width, std::vector<int64_t>* spec_kv) {
    std::vector<int> level_begin(ready.size(), 0);  // first node of the deepest level, per sequence
    for (int round = 0; round < k; ++round) {
      std::vector<int64_t> seq_ids;
      std::vector<int32_t> lens, token_ids, tree_parents;
      SampleParams sp;
      std::vector<std::pair<size_t, int>> row_owner;  // (sequence, node that the row's distribution follows; -1 = root)
      int32_t off = 0;
      for (size_t i = 0; i < ready.size(); ++i) {
        EntryRef r = ready[i];
        RequestStateEntry& e = r.e();
        ModelState& ds = e.mstates[1];
        if (!kv_[1]->Has(ds.internal_id)) kv_[1]->AddSequence(ds.internal_id);
        seq_ids.push_back(ds.internal_id);
        if (round == 0) {
          const int64_t total = r.rs->request.prompt_tokens + static_cast<int64_t>(e.committed_tokens.size());
          int64_t lag = total - kv_[1]->SequenceLength(ds.internal_id);
          if (lag > static_cast<int64_t>(e.committed_tokens.size()))
            throw std::runtime_error("Engine: draft model KV lags behind the prompt");
          for (int64_t j = static_cast<int64_t>(e.committed_tokens.size()) - lag;
               j < static_cast<int64_t>(e.committed_tokens.size()); ++j) {
            token_ids.push_back(e.committed_tokens[j].token);
            tree_parents.push_back(static_cast<int32_t>(j - (static_cast<int64_t>(e.committed_tokens.size()) - lag)) - 1);
          }
          lens.push_back(static_cast<int32_t>(lag));
          off += static_cast<int32_t>(lag);
          AddSampleRow(&sp, r, off - 1);
          row_owner.emplace_back(i, -1);
        } else {
          // drop the previous round's speculative entries, then feed the whole tree
          if ((*spec_kv)[i] > 0) kv_[1]->PopN(ds.internal_id, (*spec_kv)[i]);
          const int nodes = static_cast<int>(ds.draft_tokens.size());
          for (int j = 0; j < nodes; ++j) {
            token_ids.push_back(ds.draft_tokens[j].token);
            tree_parents.push_back(ds.draft_parents[j]);  // -1: hangs under the last committed token
          }
          lens.push_back(nodes);
          (*spec_kv)[i] = nodes;
          for (int j = level_begin[i]; j < nodes; ++j) {
            AddSampleRow(&sp, r, off + j);
            row_owner.emplace_back(i, j);
          }
          off += nodes;
        }
      }
      if (round == 0) std::fill(spec_kv->begin(), spec_kv->end(), 0);
      for (size_t row = 0; row < row_owner.size(); ++row) {
        const int slot = draft_slots_.Alloc();
        sp.prob_slots.push_back(slot);
      }
      sp.num_top_logprobs = std::max(sp.num_top_logprobs, width);
      std::vector<int64_t> embed_handles(token_ids.size(), -1);
      ForwardPlan plan = round == 0 ? kv_[1]->BeginForward(seq_ids, lens)
                                    : kv_[1]->BeginForward(seq_ids, lens, &tree_parents);
      SampleOutput out = backend_->ForwardSample(1, plan, token_ids, embed_handles, sp);
      const int num_top = sp.num_top_logprobs;
      for (size_t i = 0; i < ready.size(); ++i) level_begin[i] = static_cast<int>(ready[i].e().mstates[1].draft_tokens.size());
      for (size_t row = 0; row < row_owner.size(); ++row) {
        ModelState& ds = ready[row_owner[row].first].e().mstates[1];
        for (int c = 0; c < width; ++c) {
          SampleResult s;
          s.token = out.top_tokens[row * num_top + c];
          s.prob = out.top_probs[row * num_top + c];
          ds.draft_tokens.push_back(s);
          ds.draft_slots.push_back(sp.prob_slots[row]);
          ds.draft_parents.push_back(row_owner[row].second);
        }
      }
    }
  }

  bool StepSpecDecode() {
    std::vector<EntryRef> ready = ReadyToDecode();
    if (ready.empty()) return false;
    const int k = DraftLengthFor(static_cast<int>(ready.size()));
    if (k == 0) return StepDecode();
    int64_t max_nodes = k;  // chain; a tree of width w has w + w^2 + ... + w^k nodes
    if (cfg_.spec_tree_width > 1) {
      max_nodes = 0;
      int64_t level = 1;
      for (int d = 0; d < k; ++d) {
        level *= cfg_.spec_tree_width;
        max_nodes += level;
      }
      if (max_nodes > 63) throw std::runtime_error("Engine: spec_tree_width ^ spec_draft_length exceeds the 63-node draft tree limit");
    }
    if (!FitDecodeBatch(&ready, max_nodes + 1)) return false;
    if (static_cast<int64_t>(ready.size()) > cfg_.max_num_sequence) ready.resize(cfg_.max_num_sequence);
    // the draft model needs the same room
    {
      int64_t need = 0;
      for (auto& r : ready) need += kv_[1]->PagesNeeded(r.e().mstates[1].internal_id, max_nodes + 8);
      if (kv_[1]->NumAvailablePages() < need) return StepDecode();
    }
    const int64_t prompt_extra = 0;
    (void)prompt_extra;
    // ---- draft phase: k rounds of the small model
    double t0 = NowSeconds();
    TraceBatch(ready, "start draft");
    // Draft heads fed with the target's features grow trees the same way (reference:
    // cpp/serve/engine_actions/eagle_batch_draft.cc:38-186): the executor gives every node of an EAGLE tree its
    // parent's predicted feature, and every leaf of a Medusa tree the distribution of the head of its depth.
    const int width = std::max(1, cfg_.spec_tree_width);
    // speculative entries each sequence leaves in the draft model's KV (dropped after verification)
    std::vector<int64_t> spec_kv(ready.size(), k - 1);
    if (width > 1) DraftTree(ready, k, width, &spec_kv);
    for (int round = 0; round < (width > 1 ? 0 : k); ++round) {
      std::vector<int64_t> seq_ids;
      std::vector<int32_t> lens, token_ids;
      SampleParams sp;
      int32_t off = 0;
      for (auto& r : ready) {
        RequestStateEntry& e = r.e();
        ModelState& ds = e.mstates[1];
        if (!kv_[1]->Has(ds.internal_id)) kv_[1]->AddSequence(ds.internal_id);
        std::vector<int32_t> feed;
        if (round == 0) {
          // everything the draft model has not seen yet: lagging committed tokens
          const int64_t total = r.rs->request.prompt_tokens + static_cast<int64_t>(e.committed_tokens.size());
          const int64_t have = kv_[1]->SequenceLength(ds.internal_id);
          int64_t lag = total - have;
          if (lag > static_cast<int64_t>(e.committed_tokens.size()))
            throw std::runtime_error("Engine: draft model KV lags behind the prompt");
          for (int64_t j = static_cast<int64_t>(e.committed_tokens.size()) - lag;
               j < static_cast<int64_t>(e.committed_tokens.size()); ++j)
            feed.push_back(e.committed_tokens[j].token);
        } else {
          feed.push_back(ds.draft_tokens.back().token);
        }
        seq_ids.push_back(ds.internal_id);
        lens.push_back(static_cast<int32_t>(feed.size()));
        token_ids.insert(token_ids.end(), feed.begin(), feed.end());
        off += static_cast<int32_t>(feed.size());
        AddSampleRow(&sp, r, off - 1);
        const int slot = draft_slots_.Alloc();
        ds.draft_slots.push_back(slot);
        sp.prob_slots.push_back(slot);
      }
      std::vector<int64_t> embed_handles(token_ids.size(), -1);
      ForwardPlan plan = kv_[1]->BeginForward(seq_ids, lens);
      SampleOutput out = backend_->ForwardSample(1, plan, token_ids, embed_handles, sp);
      for (size_t i = 0; i < ready.size(); ++i) {
        ModelState& ds = ready[i].e().mstates[1];
        SampleResult s;
        s.token = out.tokens[i];
        s.prob = out.probs.empty() ? 1.f : out.probs[i];
        ds.draft_tokens.push_back(s);
        ds.draft_parents.push_back(round - 1);  // chain: node j hangs under node j-1 (-1 = root)
      }
    }
    double t1 = NowSeconds();
    metrics_.UpdateDraftTimeByBatchSize(static_cast<int>(ready.size()), t1 - t0);
    TraceBatch(ready, "finish draft");

    // ---- verify phase: one main-model pass over [last committed, drafts...]
    TraceBatch(ready, "start verify");
    std::vector<int64_t> seq_ids;
    std::vector<int32_t> lens, token_ids, tree_parents;
    VerifyParams vp;
    vp.node_indptr.push_back(0);
    int32_t off = 0;
    for (auto& r : ready) {
      RequestStateEntry& e = r.e();
      ModelState& ds = e.mstates[1];
      const int nodes = static_cast<int>(ds.draft_tokens.size());  // k for a chain, more for a tree
      seq_ids.push_back(e.mstates[0].internal_id);
      lens.push_back(nodes + 1);
      token_ids.push_back(e.committed_tokens.back().token);
      tree_parents.push_back(-1);
      vp.want_logprobs |= r.rs->request.cfg.logprobs;
      // row for the root (distribution after the last committed token)
      AddSampleRow(&vp.sampling, r, off);
      for (int j = 0; j < nodes; ++j) {
        token_ids.push_back(ds.draft_tokens[j].token);
        // chunk-local: the root is entry 0, node j is entry j + 1 and hangs under its parent's entry
        tree_parents.push_back(ds.draft_parents[j] + 1);
        vp.draft_tokens.push_back(ds.draft_tokens[j].token);
        vp.draft_prob_slots.push_back(ds.draft_slots[j]);
        vp.parents.push_back(ds.draft_parents[j]);
        vp.uniform.push_back(static_cast<float>(e.NextUniform()));
        // the row after node j: its ancestors' tokens and its own precede it
        std::vector<int32_t> path;
        for (int a = j; a >= 0; a = ds.draft_parents[a]) path.push_back(ds.draft_tokens[a].token);
        std::reverse(path.begin(), path.end());
        AddSampleRow(&vp.sampling, r, off + 1 + j, &path);
      }
      vp.node_indptr.push_back(static_cast<int32_t>(vp.draft_tokens.size()));
      vp.final_uniform.push_back(static_cast<float>(e.NextUniform()));
      off += nodes + 1;
    }
    ForwardPlan plan = kv_[0]->BeginForward(seq_ids, lens, &tree_parents);
    VerifyOutput vo = backend_->ForwardVerify(0, plan, token_ids, vp);
    for (size_t i = 0; i < ready.size(); ++i) {
      EntryRef r = ready[i];
      RequestStateEntry& e = r.e();
      ModelState& ds = e.mstates[1];
      const int beg = vo.accepted_indptr[i], end = vo.accepted_indptr[i + 1];
      const int accepted = end - beg;
      // KV: node 0 (the last committed token) is always kept; accepted draft nodes follow
      std::vector<int32_t> keep{0};
      for (int j = beg; j < end; ++j) keep.push_back(vo.accepted_nodes[j] + 1);
      const int nodes = static_cast<int>(ds.draft_tokens.size());
      std::vector<int32_t> moves = kv_[0]->CommitTreeNodes(e.mstates[0].internal_id, nodes + 1, keep);
      if (!moves.empty()) backend_->MoveKVTokens(0, moves);
      // draft KV holds [.., last committed, d_0 .. d_{k-2}]; keep the accepted part.  A feature-fed head
      // (EAGLE) computed those entries from its own predicted features: all of them are dropped and
      // the next draft phase recomputes the accepted tokens from the target's true features
      // (reference: cpp/serve/engine_actions/eagle_batch_verify.cc).
      // With a draft tree the speculative entries are dropped as well: their order in the draft KV is
      // the tree's, not the accepted path's.
      const int64_t draft_valid = (feature_fed_draft_ || width > 1) ? 0 : std::min<int64_t>(accepted, k - 1);
      if (spec_kv[i] - draft_valid > 0) kv_[1]->PopN(ds.internal_id, spec_kv[i] - draft_valid);
      // reported probabilities are the target's (the draft's own would describe another model)
      const GenerationConfig& gcfg = r.rs->request.cfg;
      auto fill_top = [&](SampleResult* s, size_t row) {
        s->top.clear();
        if (!gcfg.logprobs || vo.num_top <= 0) return;
        for (int t = 0; t < gcfg.top_logprobs && t < vo.num_top; ++t) {
          const size_t at = row * static_cast<size_t>(vo.num_top) + static_cast<size_t>(t);
          if (at < vo.top_tokens.size()) s->top.emplace_back(vo.top_tokens[at], vo.top_probs[at]);
        }
      };
      for (int j = beg; j < end; ++j) {
        SampleResult s = ds.draft_tokens[vo.accepted_nodes[j]];
        if (static_cast<size_t>(j) < vo.accepted_probs.size()) {
          s.prob = vo.accepted_probs[j];
          fill_top(&s, static_cast<size_t>(j));
        }
        CommitToken(r, s);
      }
      SampleResult fin;
      fin.token = vo.final_tokens[i];
      fin.prob = vo.final_probs.empty() ? 1.f : vo.final_probs[i];
      if (!vo.accepted_probs.empty() || vo.num_top > 0) fill_top(&fin, vo.accepted_nodes.size() + i);
      CommitToken(r, fin);
      r.rs->metrics.decode_tokens += accepted + 1;
      metrics_.spec_decode.Update(k, accepted);
      // siblings of a draft tree share their parent's slot: free every slot once
      std::sort(ds.draft_slots.begin(), ds.draft_slots.end());
      ds.draft_slots.erase(std::unique(ds.draft_slots.begin(), ds.draft_slots.end()), ds.draft_slots.end());
      for (int s : ds.draft_slots) draft_slots_.Free(s);
      ds.draft_slots.clear();
      ds.draft_tokens.clear();
      ds.draft_parents.clear();
    }
    TraceBatch(ready, "finish verify");
    ++num_verify_steps_;
    const double t2 = NowSeconds();
    metrics_.UpdateVerifyTimeByBatchSize(static_cast<int>(ready.size()), t2 - t1);
    metrics_.engine_decode_time_sum += t2 - t0;
    return true;
  }

  // ---------------------------------------------------------------- post-processing
  void FinishEntry(RequestState* rs, RequestStateEntry& e, const std::string& reason) {
    e.status = EntryStatus::kFinished;
    e.finish_reason = reason;
    --rs->num_unfinished;
  }

  void PostProcess() {
    std::vector<RequestStreamOutput> outs;
    const double now = NowSeconds();
    for (RequestState* rs : touched_) {
      if (!states_.count(rs->request.id)) continue;
      const Request& req = rs->request;
      const int n = req.cfg.n;
      RequestStreamOutput out;
      out.request_id = req.id;
      out.group_delta_token_ids.resize(n);
      out.group_delta_logprob_json_strs.resize(n);
      out.group_finish_reason.assign(n, "");
      out.group_extra_prefix_string.assign(n, "");
      bool any = false;
      for (int g = 0; g < n; ++g) {
        const int idx = n == 1 ? 0 : g + 1;
        RequestStateEntry& e = rs->entries[idx];
        if (e.status != EntryStatus::kAlive) continue;
        std::vector<int32_t>& delta = out.group_delta_token_ids[g];
        std::string finish;
        auto emit_tokens = [&](const std::vector<int32_t>& released, int64_t upto) {
          (void)upto;
          for (int32_t t : released) delta.push_back(t);
        };
        const int64_t first_new = e.next_callback_token_pos;
        while (e.next_callback_token_pos < static_cast<int64_t>(e.committed_tokens.size()) && finish.empty()) {
          const SampleResult& s = e.committed_tokens[e.next_callback_token_pos];
          ++e.next_callback_token_pos;
          if (IsStopToken(req, s.token)) {
            emit_tokens(e.stop_handler->Finish(), e.next_callback_token_pos);
            finish = "stop";
            break;
          }
          emit_tokens(e.stop_handler->Put(s.token), e.next_callback_token_pos);
          if (e.stop_handler->stop_triggered()) {
            finish = "stop";
            break;
          }
          if (e.grammar_handle >= 0 && grammar_ && grammar_->IsTerminated(e.grammar_handle)) {
            emit_tokens(e.stop_handler->Finish(), e.next_callback_token_pos);
            finish = "stop";
            break;
          }
          if (req.cfg.max_tokens >= 0 && e.next_callback_token_pos >= req.cfg.max_tokens) {
            emit_tokens(e.stop_handler->Finish(), e.next_callback_token_pos);
            finish = "length";
            break;
          }
          if (req.prompt_tokens + e.next_callback_token_pos >= cfg_.max_single_sequence_length) {
            emit_tokens(e.stop_handler->Finish(), e.next_callback_token_pos);
            finish = "length";
            break;
          }
        }
        // tokens sampled beyond a finish point (speculative decoding) are dropped
        if (!finish.empty() && e.next_callback_token_pos < static_cast<int64_t>(e.committed_tokens.size())) {
          const int64_t extra = static_cast<int64_t>(e.committed_tokens.size()) - e.next_callback_token_pos;
          rs->metrics.completion_tokens -= extra;
          e.committed_tokens.resize(e.next_callback_token_pos);
        }
        if (req.cfg.logprobs) {
          // logprob entries follow the released tokens one to one (released tokens are a suffix-
          // delayed view of the committed tokens, so walk backwards from the release point)
          const int64_t released_total = e.next_callback_token_pos;
          (void)first_new;
          int64_t start = released_total - static_cast<int64_t>(delta.size());
          if (start < 0) start = 0;
          // find where the delta tokens sit among the committed tokens
          int64_t pos = e.logprob_cursor;
          for (int32_t t : delta) {
            while (pos < static_cast<int64_t>(e.committed_tokens.size()) && e.committed_tokens[pos].token != t) ++pos;
            if (pos < static_cast<int64_t>(e.committed_tokens.size())) {
              out.group_delta_logprob_json_strs[g].push_back(LogprobJSON(tok_.get(), e.committed_tokens[pos]));
              ++pos;
            }
          }
          e.logprob_cursor = pos;
        }
        // feed the prefix cache with tokens whose KV now exists (all committed but the last)
        {
          ModelState& ms = e.mstates[0];
          int64_t without_kv = 0;  // forced tokens still waiting as inputs, else the last sampled token
          for (auto& in : ms.inputs) without_kv += in.Length();
          const int64_t with_kv = static_cast<int64_t>(e.committed_tokens.size()) - std::max<int64_t>(1, without_kv);
          if (prefix_cache_.HasSequence(ms.internal_id) && with_kv > ms.cached_committed_tokens && finish.empty()) {
            std::vector<int32_t> toks;
            for (int64_t j = ms.cached_committed_tokens; j < with_kv; ++j) toks.push_back(e.committed_tokens[j].token);
            prefix_cache_.ExtendSequence(ms.internal_id, toks);
            ms.cached_committed_tokens = with_kv;
          }
        }
        if (!e.extra_prefix_string.empty()) {
          out.group_extra_prefix_string[g] = std::move(e.extra_prefix_string);
          e.extra_prefix_string.clear();
          any = true;
        }
        if (!delta.empty()) any = true;
        if (!finish.empty()) {
          any = true;
          out.group_finish_reason[g] = finish;
          if (req.cfg.debug_config.disagg_config.kind == DisaggRequestKind::kRemoteSend)
            SendKVOfFinishedEntry(rs, e);
          FinishEntry(rs, e, finish);
          // the KV may hold tokens past the finish point (speculation): trim, then recycle
          ReleaseEntry(e, /*recycle=*/true);
        }
      }
      if (rs->num_unfinished == 0) {
        rs->metrics.finish_time = now;
        if (!rs->prefill_done) rs->metrics.prefill_end_time = now;
        out.request_final_usage_json_str = rs->metrics.AsUsageJSON(true).dump();
        metrics_.RequestFinishUpdate(rs->metrics);
        for (auto& e : rs->entries) ReleaseEntry(e, /*recycle=*/true);
        any = true;
      }
      if (any) outs.push_back(std::move(out));
      if (rs->num_unfinished == 0) {
        Trace(req.id, "finish");
        RemoveFromQueues(rs);
        ForgetInflight(rs);
        states_.erase(req.id);
      }
    }
    prefix_cache_.CommitSequenceExtention();
    touched_.clear();
    Emit(std::move(outs));
  }

  EngineConfig cfg_;
  std::vector<EngineModelInfo> models_;
  std::shared_ptr<ModelBackend> backend_;
  std::shared_ptr<const Tokenizer> tok_;
  std::shared_ptr<GrammarBackend> grammar_;
  std::shared_ptr<EventTraceRecorder> trace_;
  StreamCallback callback_;
  PrefixCache prefix_cache_;
  std::vector<std::unique_ptr<KVManager>> kv_;
  GenerationConfig default_gen_;
  std::unordered_map<std::string, std::unique_ptr<RequestState>> states_;
  std::vector<RequestState*> running_, waiting_, touched_;
  IdManager ids_;
  SlotManager draft_slots_;
  EngineMetrics metrics_;
  std::mt19937_64 seed_rng_;
  double t_assemble_ = 0, t_plan_ = 0, t_backend_ = 0, t_commit_ = 0, t_post_ = 0;
  bool spec_ = false;
  bool pipelined_decode_ = true;   // MLCB_PIPELINED_DECODE=0 switches the deferred-read decode path off
  bool pipelined_pause_ = false;   // one ordinary step is due (memory pressure) before pipelining resumes
  InflightDecode inflight_;
  bool feature_fed_draft_ = false;  // EAGLE / Medusa: the draft head consumes the target's hidden states
  int64_t num_prefill_steps_ = 0, num_decode_steps_ = 0, num_verify_steps_ = 0, num_preemptions_ = 0;
  int64_t num_pipelined_steps_ = 0, num_dropped_tokens_ = 0;
};

// ====================================================================== mock echo engine
class MockEchoEngine : public Engine {
 public:
  MockEchoEngine(EngineConfig cfg, std::string model_config_json, std::shared_ptr<const Tokenizer> tok,
                 StreamCallback cb)
      : cfg_(std::move(cfg)), tok_(std::move(tok)), callback_(std::move(cb)) {
    if (!model_config_json.empty()) {
      Value v = json::parse(model_config_json);
      if (v.is_object()) default_gen_ = GenerationConfig::DefaultsFromModelConfig(v.as_object());
    }
    if (cfg_.max_single_sequence_length <= 0) cfg_.max_single_sequence_length = 1 << 20;
  }
  void SetStreamCallback(StreamCallback cb) override { callback_ = std::move(cb); }
  const GenerationConfig& DefaultGenerationConfig() const override { return default_gen_; }
  const EngineConfig& Config() const override { return cfg_; }
  bool Empty() const override { return pending_.empty(); }
  void Reset() override { pending_.clear(); }
  std::string JSONMetrics() const override { return metrics_.AsJSON().dump(); }
  void AddRequest(Request r) override {
    State st;
    for (auto& in : r.inputs) st.prompt.insert(st.prompt.end(), in.tokens.begin(), in.tokens.end());
    st.req = std::move(r);
    st.metrics.prompt_tokens = static_cast<int64_t>(st.prompt.size());
    st.metrics.add_time = NowSeconds();
    pending_.push_back(std::move(st));
  }
  void AbortRequest(const std::string& id) override {
    pending_.erase(std::remove_if(pending_.begin(), pending_.end(), [&](const State& s) { return s.req.id == id; }),
                   pending_.end());
  }
  void AbortAllRequests() override { pending_.clear(); }
  void Step() override {
    // one token per request per step, so streaming and abort behave like a real engine
    std::vector<RequestStreamOutput> outs;
    for (auto& st : pending_) {
      const int n = st.req.cfg.n;
      RequestStreamOutput out;
      out.request_id = st.req.id;
      out.group_delta_token_ids.resize(n);
      out.group_delta_logprob_json_strs.resize(n);
      out.group_finish_reason.assign(n, "");
      out.group_extra_prefix_string.assign(n, "");
      const int64_t limit = st.req.cfg.max_tokens >= 0
                                ? std::min<int64_t>(st.req.cfg.max_tokens, static_cast<int64_t>(st.prompt.size()))
                                : static_cast<int64_t>(st.prompt.size());
      if (st.pos == 0) st.metrics.prefill_end_time = NowSeconds();
      if (st.pos < limit) {
        for (int g = 0; g < n; ++g) out.group_delta_token_ids[g].push_back(st.prompt[st.pos]);
        ++st.pos;
        st.metrics.completion_tokens += 1;
      }
      if (st.pos >= limit) {
        const bool by_len = st.req.cfg.max_tokens >= 0 && st.req.cfg.max_tokens <= static_cast<int64_t>(st.prompt.size());
        out.group_finish_reason.assign(n, by_len ? "length" : "stop");
        st.metrics.finish_time = NowSeconds();
        st.metrics.prefill_tokens = st.metrics.prompt_tokens;
        st.metrics.decode_tokens = st.metrics.completion_tokens;
        Value usage = st.metrics.AsUsageJSON(true);
        // the echo engine reports the parsed generation config for API-plumbing tests
        usage.as_object()["extra"] = st.req.cfg.AsJSON();
        out.request_final_usage_json_str = usage.dump();
        metrics_.RequestFinishUpdate(st.metrics);
        st.done = true;
      }
      outs.push_back(std::move(out));
    }
    pending_.erase(std::remove_if(pending_.begin(), pending_.end(), [](const State& s) { return s.done; }),
                   pending_.end());
    if (callback_ && !outs.empty()) callback_(std::move(outs));
  }

 private:
  struct State {
    Request req;
    std::vector<int32_t> prompt;
    int64_t pos = 0;
    bool done = false;
    RequestMetrics metrics;
  };
  EngineConfig cfg_;
  std::shared_ptr<const Tokenizer> tok_;
  StreamCallback callback_;
  GenerationConfig default_gen_;
  std::vector<State> pending_;
  EngineMetrics metrics_;
};

}  // namespace

std::unique_ptr<Engine> Engine::Create(EngineConfig config, std::vector<EngineModelInfo> models,
                                       std::shared_ptr<ModelBackend> backend,
                                       std::shared_ptr<const Tokenizer> tokenizer,
                                       std::shared_ptr<GrammarBackend> grammar,
                                       std::shared_ptr<EventTraceRecorder> trace, StreamCallback callback) {
  return std::make_unique<EngineImpl>(std::move(config), std::move(models), std::move(backend),
                                      std::move(tokenizer), std::move(grammar), std::move(trace),
                                      std::move(callback));
}

std::unique_ptr<Engine> Engine::CreateMockEcho(EngineConfig config, std::string model_config_json,
                                               std::shared_ptr<const Tokenizer> tokenizer,
                                               StreamCallback callback) {
  return std::make_unique<MockEchoEngine>(std::move(config), std::move(model_config_json),
                                          std::move(tokenizer), std::move(callback));
}

}  // namespace mlcb
