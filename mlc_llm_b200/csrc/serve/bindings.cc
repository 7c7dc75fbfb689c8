// pybind11 bindings of the serving runtime (module `mlc_llm_b200._core`).
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "config.h"
#include "conv_template.h"
#include "engine.h"
#include "json_ffi_engine.h"
#include "kv_manager.h"
#include "metrics.h"
#include "prefix_cache.h"
#include "radix_tree.h"
#include "sampler.h"
#include "tokenizer.h"

namespace py = pybind11;
using namespace mlcb;

namespace {

template <typename T>
py::array_t<T> ToArray(const std::vector<T>& v) {
  return py::array_t<T>(static_cast<py::ssize_t>(v.size()), v.data());
}

template <typename T>
std::vector<T> FromArray(const py::object& o) {
  if (o.is_none()) return {};
  auto arr = py::array_t<T, py::array::c_style | py::array::forcecast>::ensure(o);
  if (!arr) throw std::runtime_error("expected a numeric array");
  return std::vector<T>(arr.data(), arr.data() + arr.size());
}

py::dict PlanToDict(const ForwardPlan& p) {
  py::dict d;
  d["seq_ids"] = ToArray(p.seq_ids);
  d["append_lens"] = ToArray(p.append_lens);
  d["seq_lens"] = ToArray(p.seq_lens);
  d["page_indptr"] = ToArray(p.page_indptr);
  d["page_indices"] = ToArray(p.page_indices);
  d["q_indptr"] = ToArray(p.q_indptr);
  d["positions"] = ToArray(p.positions);
  d["slots"] = ToArray(p.slots);
  d["q_seq"] = ToArray(p.q_seq);
  d["q_kvlen"] = ToArray(p.q_kvlen);
  d["q_kvstart"] = ToArray(p.q_kvstart);
  d["tree_mask"] = ToArray(p.tree_mask);
  d["page_copies"] = ToArray(p.page_copies);
  d["seq_forks"] = ToArray(p.seq_forks);
  d["max_append"] = p.max_append;
  d["max_seq_len"] = p.max_seq_len;
  return d;
}

py::dict SampleParamsToDict(const SampleParams& s) {
  py::dict d;
  d["logit_token_index"] = ToArray(s.logit_token_index);
  d["temperature"] = ToArray(s.temperature);
  d["top_p"] = ToArray(s.top_p);
  d["top_k"] = ToArray(s.top_k);
  d["uniform"] = ToArray(s.uniform);
  d["penalties"] = ToArray(s.penalties);
  d["pen_row"] = ToArray(s.pen_row);
  d["pen_token"] = ToArray(s.pen_token);
  d["pen_count"] = ToArray(s.pen_count);
  d["bias_row"] = ToArray(s.bias_row);
  d["bias_token"] = ToArray(s.bias_token);
  d["bias_value"] = ToArray(s.bias_value);
  d["mask_rows"] = ToArray(s.mask_rows);
  d["mask_bits"] = ToArray(s.mask_bits);
  d["num_top_logprobs"] = s.num_top_logprobs;
  d["prob_slots"] = ToArray(s.prob_slots);
  return d;
}

class PyModelBackend : public ModelBackend {
 public:
  explicit PyModelBackend(py::object impl) : impl_(std::move(impl)) {}
  ~PyModelBackend() override {
    py::gil_scoped_acquire gil;
    impl_ = py::object();
  }
  SampleOutput ForwardSample(int model_id, const ForwardPlan& plan, const std::vector<int32_t>& token_ids,
                             const std::vector<int64_t>& embed_handles, const SampleParams& sampling) override {
    py::gil_scoped_acquire gil;
    bool any_embed = false;
    for (int64_t h : embed_handles) any_embed |= h >= 0;
    py::object res = impl_.attr("forward_sample")(model_id, PlanToDict(plan), ToArray(token_ids),
                                                  any_embed ? py::object(ToArray(embed_handles)) : py::none(),
                                                  SampleParamsToDict(sampling));
    SampleOutput out;
    if (res.is_none()) return out;
    py::dict d = res.cast<py::dict>();
    out.tokens = FromArray<int32_t>(d["tokens"]);
    if (d.contains("probs")) out.probs = FromArray<float>(d["probs"]);
    if (d.contains("top_tokens")) out.top_tokens = FromArray<int32_t>(d["top_tokens"]);
    if (d.contains("top_probs")) out.top_probs = FromArray<float>(d["top_probs"]);
    return out;
  }
  static SampleOutput SampleFromDict(const py::object& res) {
    SampleOutput out;
    if (res.is_none()) return out;
    py::dict d = res.cast<py::dict>();
    out.tokens = FromArray<int32_t>(d["tokens"]);
    if (d.contains("probs")) out.probs = FromArray<float>(d["probs"]);
    if (d.contains("top_tokens")) out.top_tokens = FromArray<int32_t>(d["top_tokens"]);
    if (d.contains("top_probs")) out.top_probs = FromArray<float>(d["top_probs"]);
    return out;
  }
  bool LaunchSample(int model_id, const ForwardPlan& plan, const std::vector<int32_t>& token_ids,
                    const std::vector<int32_t>& token_src, const SampleParams& sampling) override {
    py::gil_scoped_acquire gil;
    if (!py::hasattr(impl_, "forward_sample_launch")) return false;
    return impl_.attr("forward_sample_launch")(model_id, PlanToDict(plan), ToArray(token_ids), ToArray(token_src),
                                               SampleParamsToDict(sampling)).cast<bool>();
  }
  SampleOutput WaitSample(int model_id) override {
    py::gil_scoped_acquire gil;
    return SampleFromDict(impl_.attr("forward_sample_wait")(model_id));
  }
  VerifyOutput ForwardVerify(int model_id, const ForwardPlan& plan, const std::vector<int32_t>& token_ids,
                             const VerifyParams& v) override {
    py::gil_scoped_acquire gil;
    py::dict vd;
    vd["node_indptr"] = ToArray(v.node_indptr);
    vd["draft_tokens"] = ToArray(v.draft_tokens);
    vd["draft_prob_slots"] = ToArray(v.draft_prob_slots);
    vd["parents"] = ToArray(v.parents);
    vd["want_logprobs"] = v.want_logprobs;
    vd["uniform"] = ToArray(v.uniform);
    vd["final_uniform"] = ToArray(v.final_uniform);
    vd["sampling"] = SampleParamsToDict(v.sampling);
    py::dict d = impl_.attr("forward_verify")(model_id, PlanToDict(plan), ToArray(token_ids), vd).cast<py::dict>();
    VerifyOutput out;
    out.accepted_indptr = FromArray<int32_t>(d["accepted_indptr"]);
    out.accepted_nodes = FromArray<int32_t>(d["accepted_nodes"]);
    out.final_tokens = FromArray<int32_t>(d["final_tokens"]);
    if (d.contains("final_probs")) out.final_probs = FromArray<float>(d["final_probs"]);
    if (d.contains("accepted_probs")) out.accepted_probs = FromArray<float>(d["accepted_probs"]);
    if (d.contains("top_tokens")) out.top_tokens = FromArray<int32_t>(d["top_tokens"]);
    if (d.contains("top_probs")) out.top_probs = FromArray<float>(d["top_probs"]);
    if (d.contains("num_top")) out.num_top = d["num_top"].cast<int32_t>();
    return out;
  }
  void MoveKVTokens(int model_id, const std::vector<int32_t>& moves) override {
    py::gil_scoped_acquire gil;
    impl_.attr("move_kv_tokens")(model_id, ToArray(moves));
  }
  void ApplyPageCopies(int model_id, const std::vector<int32_t>& copies) override {
    py::gil_scoped_acquire gil;
    impl_.attr("apply_page_copies")(model_id, ToArray(copies));
  }
  void SendKV(int model_id, const std::vector<int32_t>& src_slots, const std::string& metadata) override {
    py::gil_scoped_acquire gil;
    impl_.attr("send_kv")(model_id, ToArray(src_slots), metadata);
  }
  void Synchronize() override {
    py::gil_scoped_acquire gil;
    if (py::hasattr(impl_, "synchronize")) impl_.attr("synchronize")();
  }
  void ReleaseEmbedding(int64_t handle) override {
    py::gil_scoped_acquire gil;
    if (py::hasattr(impl_, "release_embedding")) impl_.attr("release_embedding")(handle);
  }
  void Reset() override {
    py::gil_scoped_acquire gil;
    if (py::hasattr(impl_, "reset")) impl_.attr("reset")();
  }

 private:
  py::object impl_;
};

class PyGrammarBackend : public GrammarBackend {
 public:
  explicit PyGrammarBackend(py::object impl) : impl_(std::move(impl)) {}
  ~PyGrammarBackend() override {
    py::gil_scoped_acquire gil;
    impl_ = py::object();
  }
  int64_t Create(const std::string& rf) override {
    py::gil_scoped_acquire gil;
    return impl_.attr("create")(rf).cast<int64_t>();
  }
  void Release(int64_t h) override {
    py::gil_scoped_acquire gil;
    impl_.attr("release")(h);
  }
  std::vector<int32_t> NextTokenBitmask(int64_t h) override {
    py::gil_scoped_acquire gil;
    return FromArray<int32_t>(impl_.attr("next_token_bitmask")(h));
  }
  bool AcceptToken(int64_t h, int32_t t) override {
    py::gil_scoped_acquire gil;
    return impl_.attr("accept_token")(h, t).cast<bool>();
  }
  void Rollback(int64_t h, int n) override {
    py::gil_scoped_acquire gil;
    impl_.attr("rollback")(h, n);
  }
  bool IsTerminated(int64_t h) override {
    py::gil_scoped_acquire gil;
    return impl_.attr("is_terminated")(h).cast<bool>();
  }
  std::string FindJumpForwardString(int64_t h) override {
    py::gil_scoped_acquire gil;
    return impl_.attr("find_jump_forward_string")(h).cast<std::string>();
  }

 private:
  py::object impl_;
};

Request MakeRequest(const std::string& id, const py::list& inputs, const GenerationConfig& cfg) {
  Request r;
  r.id = id;
  r.cfg = cfg;
  for (auto item : inputs) {
    InputItem in;
    if (py::isinstance<py::tuple>(item)) {
      // ("embed", handle, length)
      py::tuple t = item.cast<py::tuple>();
      in.kind = 1;
      in.embed_handle = t[1].cast<int64_t>();
      in.embed_len = t[2].cast<int32_t>();
    } else {
      in.tokens = FromArray<int32_t>(py::reinterpret_borrow<py::object>(item));
    }
    r.inputs.push_back(std::move(in));
  }
  return r;
}

// One field of a stream output as a Python object. Outputs cross into Python as thin wrappers and are
// converted field by field on access: a decode step of a large batch emits hundreds of them, and most
// consumers read one or two fields.
py::object OutputField(const RequestStreamOutput& o, const std::string& key) {
  if (key == "request_id") return py::str(o.request_id);
  if (key == "group_delta_token_ids") return py::cast(o.group_delta_token_ids);
  if (key == "group_delta_logprob_json_strs") return py::cast(o.group_delta_logprob_json_strs);
  if (key == "group_finish_reason") {
    py::list fr;
    for (auto& s : o.group_finish_reason) fr.append(s.empty() ? py::object(py::none()) : py::object(py::str(s)));
    return std::move(fr);
  }
  if (key == "group_extra_prefix_string") return py::cast(o.group_extra_prefix_string);
  if (key == "text_is_final") return py::bool_(o.text_is_final);
  if (key == "request_final_usage_json_str")
    return o.request_final_usage_json_str.empty() ? py::object(py::none())
                                                  : py::object(py::str(o.request_final_usage_json_str));
  throw py::key_error(key);
}

const char* const kOutputKeys[] = {"request_id", "group_delta_token_ids", "group_delta_logprob_json_strs",
                                   "group_finish_reason", "group_extra_prefix_string",
                                   "request_final_usage_json_str", "text_is_final"};

StreamCallback WrapCallback(py::object fn) {
  if (fn.is_none()) return nullptr;
  auto holder = std::make_shared<py::object>(std::move(fn));
  return [holder](std::vector<RequestStreamOutput> outs) {
    py::gil_scoped_acquire gil;
    py::list lst;
    for (auto& o : outs) lst.append(py::cast(std::move(o)));
    (*holder)(lst);
  };
}

std::shared_ptr<Tokenizer> MakeTokenizer(std::vector<std::string> vocab, const std::string& info_json,
                                         py::object encode, std::vector<int32_t> special) {
  Tokenizer::EncodeFn fn = nullptr;
  if (!encode.is_none()) {
    auto holder = std::make_shared<py::object>(std::move(encode));
    fn = [holder](const std::string& text) {
      py::gil_scoped_acquire gil;
      return FromArray<int32_t>((*holder)(text));
    };
  }
  return std::make_shared<Tokenizer>(std::move(vocab), TokenizerInfo::FromJSON(info_json), std::move(fn),
                                     std::move(special));
}

std::vector<EngineModelInfo> ParseModelInfos(const py::list& models) {
  std::vector<EngineModelInfo> out;
  for (auto m : models) {
    py::dict d = m.cast<py::dict>();
    EngineModelInfo info;
    info.vocab_size = d["vocab_size"].cast<int64_t>();
    info.num_pages = d["num_pages"].cast<int64_t>();
    info.eos_token_ids = d["eos_token_ids"].cast<std::vector<int32_t>>();
    info.generation_defaults_json = d["model_config_json"].cast<std::string>();
    out.push_back(std::move(info));
  }
  return out;
}

// Forwards to an Engine owned by a Python object (kept alive by the proxy).
class ProxyEngine : public Engine {
 public:
  ProxyEngine(py::object owner, Engine* impl) : owner_(std::move(owner)), impl_(impl) {}
  ~ProxyEngine() override {
    py::gil_scoped_acquire gil;
    owner_ = py::object();
  }
  void AddRequest(Request r) override { impl_->AddRequest(std::move(r)); }
  void AbortRequest(const std::string& id) override { impl_->AbortRequest(id); }
  void AbortAllRequests() override { impl_->AbortAllRequests(); }
  void Step() override { impl_->Step(); }
  bool Empty() const override { return impl_->Empty(); }
  void Reset() override { impl_->Reset(); }
  std::string JSONMetrics() const override { return impl_->JSONMetrics(); }
  const GenerationConfig& DefaultGenerationConfig() const override { return impl_->DefaultGenerationConfig(); }
  const EngineConfig& Config() const override { return impl_->Config(); }
  void SetStreamCallback(StreamCallback cb) override { impl_->SetStreamCallback(std::move(cb)); }
  std::string DebugStats() const override { return impl_->DebugStats(); }

 private:
  py::object owner_;
  Engine* impl_;
};

}  // namespace

PYBIND11_MODULE(_core, m) {
  // ---------------------------------------------------------------- stream outputs (dict-like, lazy)
  py::class_<RequestStreamOutput>(m, "StreamOutput")
      .def("__getitem__", [](const RequestStreamOutput& o, const std::string& key) { return OutputField(o, key); })
      .def("__contains__", [](const RequestStreamOutput&, const std::string& key) {
        for (const char* k : kOutputKeys)
          if (key == k) return true;
        return false;
      })
      .def("get", [](const RequestStreamOutput& o, const std::string& key, py::object dflt) {
        for (const char* k : kOutputKeys)
          if (key == k) return OutputField(o, key);
        return dflt;
      }, py::arg("key"), py::arg("default") = py::none())
      .def("keys", []() {
        py::list out;
        for (const char* k : kOutputKeys) out.append(py::str(k));
        return out;
      })
      .def("asdict", [](const RequestStreamOutput& o) {
        py::dict d;
        for (const char* k : kOutputKeys) d[py::str(k)] = OutputField(o, k);
        return d;
      });

  m.doc() = "Native serving runtime of mlc_llm_b200";

  // ---------------------------------------------------------------- radix tree / prefix cache
  py::class_<RadixTree>(m, "PagedRadixTree")
      .def(py::init<int64_t>(), py::arg("max_blocks") = 1 << 16)
      .def("match",
           [](const RadixTree& t, const std::vector<int32_t>& tokens) {
             auto r = t.Match(tokens);
             return py::make_tuple(r.first, py::tuple(py::cast(r.second)));
           })
      .def("add", &RadixTree::Add)
      .def("remove", &RadixTree::Remove)
      .def("extend", &RadixTree::Extend)
      .def("rollback", &RadixTree::Rollback)
      .def("fork", &RadixTree::Fork)
      .def("get", &RadixTree::Get)
      .def("get_length", &RadixTree::GetLength)
      .def("has", &RadixTree::Has)
      .def("free_capacity", &RadixTree::FreeCapacity);

  py::class_<PrefixMatch>(m, "PrefixMatch")
      .def_readonly("prefilled_offset", &PrefixMatch::prefilled_offset)
      .def_readonly("forked_seq_id", &PrefixMatch::forked_seq_id)
      .def_readonly("reused_seq_id", &PrefixMatch::reused_seq_id)
      .def_readonly("reused_seq_pop_last_tokens", &PrefixMatch::reused_seq_pop_last_tokens);

  py::class_<PrefixCache>(m, "PrefixCache")
      .def(py::init([](bool enabled, int64_t max_recycling, py::object cb) {
             PrefixCache::RemoveCallback fn = nullptr;
             if (!cb.is_none()) {
               auto holder = std::make_shared<py::object>(std::move(cb));
               fn = [holder](int64_t id) { (*holder)(id); };
             }
             return new PrefixCache(enabled, max_recycling, fn);
           }),
           py::arg("enabled") = true, py::arg("max_recycling") = -1, py::arg("remove_callback") = py::none())
      .def("insert_sequence", &PrefixCache::InsertSequence, py::arg("seq_id"), py::arg("tokens"),
           py::arg("sliding_window_size") = -1, py::arg("attention_sink_size") = 0)
      .def("extend_sequence", &PrefixCache::ExtendSequence)
      .def("commit_sequence_extention", &PrefixCache::CommitSequenceExtention)
      .def("rollback_sequence", &PrefixCache::RollBackSequence)
      .def("recycle_sequence", &PrefixCache::RecycleSequence, py::arg("seq_id"), py::arg("lazy") = true)
      .def("try_free_memory", &PrefixCache::TryFreeMemory)
      .def("has_sequence", &PrefixCache::HasSequence)
      .def("num_recycling", &PrefixCache::NumRecycling)
      .def("reset", &PrefixCache::Reset);

  // ---------------------------------------------------------------- KV manager
  py::class_<KVManager>(m, "KVManager")
      .def(py::init<int64_t, int, int64_t>(), py::arg("num_pages"), py::arg("page_size") = 16,
           py::arg("max_num_sequence") = 1 << 20)
      .def("clear", &KVManager::Clear)
      .def("add_sequence", &KVManager::AddSequence)
      .def("fork_sequence", &KVManager::ForkSequence, py::arg("parent_id"), py::arg("child_id"),
           py::arg("fork_pos") = -1)
      .def("remove_sequence", &KVManager::RemoveSequence)
      .def("popn", &KVManager::PopN)
      .def("enable_sliding_window", &KVManager::EnableSlidingWindow)
      .def("has", &KVManager::Has)
      .def("sequence_length", &KVManager::SequenceLength)
      .def("sequence_pages", &KVManager::SequencePages)
      .def("begin_forward",
           [](KVManager& kv, const std::vector<int64_t>& ids, const std::vector<int32_t>& lens,
              py::object tree_parents) {
             if (tree_parents.is_none()) return PlanToDict(kv.BeginForward(ids, lens));
             std::vector<int32_t> tp = FromArray<int32_t>(tree_parents);
             return PlanToDict(kv.BeginForward(ids, lens, &tp));
           },
           py::arg("seq_ids"), py::arg("append_lens"), py::arg("tree_parents") = py::none())
      .def("commit_tree_nodes", &KVManager::CommitTreeNodes)
      .def("pages_needed", &KVManager::PagesNeeded)
      .def("num_available_pages", &KVManager::NumAvailablePages)
      .def("total_sequence_length", &KVManager::TotalSequenceLength)
      .def("num_pages", &KVManager::NumPages)
      .def("num_sequences", &KVManager::NumSequences);

  // ---------------------------------------------------------------- tokenizer glue
  m.def("detect_tokenizer_info", [](const std::string& tokenizer_json) {
    return TokenizerInfo::Detect(tokenizer_json).AsJSON();
  });
  m.def("post_process_token", [](const std::string& tok, const std::string& method) {
    return py::bytes(PostProcessToken(tok, method));
  });
  py::class_<Tokenizer, std::shared_ptr<Tokenizer>>(m, "Tokenizer")
      .def(py::init(&MakeTokenizer), py::arg("vocab"), py::arg("info_json"), py::arg("encode") = py::none(),
           py::arg("special_token_ids") = std::vector<int32_t>())
      .def("encode", &Tokenizer::Encode)
      .def("encode_no_prepend_space", &Tokenizer::EncodeNoPrependSpace)
      .def("prefix_token_mask", [](const Tokenizer& t) {
        const std::vector<bool>& m = t.PrefixTokenMask();
        return std::vector<int>(m.begin(), m.end());
      })
      .def("decode", [](const Tokenizer& t, const std::vector<int32_t>& ids) { return t.Decode(ids); })
      .def("token_bytes", [](const Tokenizer& t, int32_t id) { return py::bytes(t.TokenBytes(id)); })
      .def("vocab_size", &Tokenizer::VocabSize)
      .def("token_to_id", &Tokenizer::TokenToId)
      .def("id_to_token", &Tokenizer::IdToRawToken)
      .def("info_json", [](const Tokenizer& t) { return t.info().AsJSON(); })
      .def("post_processed_token_table", [](const Tokenizer& t) {
        py::list out;
        for (auto& s : t.PostprocTokenTable()) out.append(py::bytes(s));
        return out;
      });
  py::class_<TextStreamer>(m, "TextStreamer")
      .def(py::init<std::shared_ptr<const Tokenizer>>())
      .def("put", &TextStreamer::Put)
      .def("finish", &TextStreamer::Finish);
  py::class_<StopStrHandler>(m, "StopStrHandler")
      .def(py::init<std::vector<std::string>, std::shared_ptr<const Tokenizer>>())
      .def("put", &StopStrHandler::Put)
      .def("finish", &StopStrHandler::Finish)
      .def_property_readonly("stop_triggered", &StopStrHandler::stop_triggered);

  // ---------------------------------------------------------------- tracing / config
  py::class_<EventTraceRecorder, std::shared_ptr<EventTraceRecorder>>(m, "EventTraceRecorder")
      .def(py::init<>())
      .def("add_event", py::overload_cast<const std::string&, const std::string&>(&EventTraceRecorder::AddEvent))
      .def("add_event_batch",
           py::overload_cast<const std::vector<std::string>&, const std::string&>(&EventTraceRecorder::AddEvent))
      .def("dump_json", &EventTraceRecorder::DumpJSON)
      .def("clear", &EventTraceRecorder::Clear);

  py::class_<GenerationConfig>(m, "GenerationConfig")
      .def_static("from_json",
                  [](const std::string& s, const std::string& defaults_model_config_json) {
                    GenerationConfig d;
                    if (!defaults_model_config_json.empty()) {
                      json::Value v = json::parse(defaults_model_config_json);
                      if (v.is_object()) d = GenerationConfig::DefaultsFromModelConfig(v.as_object());
                    }
                    return GenerationConfig::FromJSON(s, d);
                  },
                  py::arg("json_str"), py::arg("model_config_json") = "")
      .def("as_json", [](const GenerationConfig& g) { return g.AsJSON().dump(); })
      .def_readonly("n", &GenerationConfig::n)
      .def_readonly("max_tokens", &GenerationConfig::max_tokens);

  m.def("engine_config_roundtrip", [](const std::string& s) { return EngineConfig::FromJSON(s).AsJSON().dump(); });
  m.def(
      "infer_capacity",
      [](const std::string& engine_config_json, const py::list& models, int64_t gpu_total_bytes) {
        EngineConfig cfg = EngineConfig::FromJSON(engine_config_json);
        std::vector<ModelCapacityInfo> infos;
        for (auto mm : models) {
          py::dict d = mm.cast<py::dict>();
          ModelCapacityInfo mi;
          auto geti = [&](const char* k, int64_t dflt) { return d.contains(k) ? d[k].cast<int64_t>() : dflt; };
          mi.params_bytes = geti("params_bytes", 0);
          mi.num_layers = geti("num_layers", 0);
          mi.num_qo_heads = geti("num_qo_heads", 0);
          mi.num_kv_heads = geti("num_kv_heads", 0);
          mi.head_dim = geti("head_dim", 0);
          mi.vocab_size = geti("vocab_size", 0);
          mi.context_window_size = geti("context_window_size", -1);
          mi.sliding_window_size = geti("sliding_window_size", -1);
          mi.prefill_chunk_size = geti("prefill_chunk_size", 2048);
          mi.max_batch_size = geti("max_batch_size", 128);
          mi.pipeline_parallel_stages = static_cast<int>(geti("pipeline_parallel_stages", 1));
          mi.kv_bytes_per_element = static_cast<int>(geti("kv_bytes_per_element", 2));
          mi.rnn_state_bytes_per_sequence = geti("rnn_state_bytes_per_sequence", 0);
          mi.hidden_size = geti("hidden_size", 0);
          infos.push_back(mi);
        }
        CapacityResult r = cfg.kv_state_kind == "rnn_state" ? InferRNNStateCapacity(cfg, infos, gpu_total_bytes)
                                                            : InferCapacity(cfg, infos, gpu_total_bytes);
        py::dict out;
        out["config_json"] = r.config.AsJSON().dump();
        out["num_pages"] = r.num_pages;
        out["kv_bytes_per_token"] = r.kv_bytes_per_token;
        out["report"] = r.report;
        return out;
      },
      py::arg("engine_config_json"), py::arg("models"), py::arg("gpu_total_bytes"));

  // ---------------------------------------------------------------- CPU sampler
  m.def("cpu_sample_top_p", [](py::array_t<float, py::array::c_style | py::array::forcecast> prob, double top_p,
                               double uniform) {
    auto r = SampleTopPFromProb(prob.data(), static_cast<int64_t>(prob.size()), top_p, uniform);
    return py::make_tuple(r.first, r.second);
  });
  m.def("cpu_renormalize_top_p", [](py::array_t<float, py::array::c_style> prob, double top_p) {
    RenormalizeProbByTopP(prob.mutable_data(), static_cast<int64_t>(prob.size()), top_p);
  });
  m.def("cpu_verify_chain", [](py::array_t<float, py::array::c_style> model_probs,
                               py::array_t<float, py::array::c_style | py::array::forcecast> draft_probs,
                               const std::vector<int32_t>& draft_tokens, const std::vector<double>& uniforms,
                               double final_uniform) {
    const int64_t vocab = model_probs.shape(1);
    auto r = VerifyDraftChain(model_probs.mutable_data(), draft_probs.data(), draft_tokens, uniforms, final_uniform, vocab);
    return py::make_tuple(r.first, r.second);
  });

  // ---------------------------------------------------------------- conversation template (C++)
  m.def("conv_template_render", [](const std::string& conv_json, const std::string& messages_json) {
    return RenderConversation(conv_json, messages_json);
  });

  // ---------------------------------------------------------------- engines
  py::class_<Engine>(m, "Engine")
      .def_static(
          "create",
          [](const std::string& engine_config_json, const py::list& models, py::object backend,
             std::shared_ptr<Tokenizer> tokenizer, py::object grammar, std::shared_ptr<EventTraceRecorder> trace,
             py::object callback) {
            std::shared_ptr<GrammarBackend> gb;
            if (!grammar.is_none()) gb = std::make_shared<PyGrammarBackend>(grammar);
            return Engine::Create(EngineConfig::FromJSON(engine_config_json), ParseModelInfos(models),
                                  std::make_shared<PyModelBackend>(backend), tokenizer, gb, trace,
                                  WrapCallback(callback));
          },
          py::arg("engine_config_json"), py::arg("models"), py::arg("backend"), py::arg("tokenizer"),
          py::arg("grammar") = py::none(), py::arg("trace") = nullptr, py::arg("callback") = py::none())
      .def_static(
          "create_mock_echo",
          [](const std::string& engine_config_json, const std::string& model_config_json,
             std::shared_ptr<Tokenizer> tokenizer, py::object callback) {
            return Engine::CreateMockEcho(EngineConfig::FromJSON(engine_config_json), model_config_json, tokenizer,
                                          WrapCallback(callback));
          })
      .def("add_request",
           [](Engine& e, const std::string& id, const py::list& inputs, const std::string& gen_cfg_json) {
             GenerationConfig g = GenerationConfig::FromJSON(gen_cfg_json, e.DefaultGenerationConfig());
             e.AddRequest(MakeRequest(id, inputs, g));
           })
      .def("abort_request", &Engine::AbortRequest)
      .def("abort_all_requests", &Engine::AbortAllRequests)
      .def("step", &Engine::Step, py::call_guard<py::gil_scoped_release>())
      .def("empty", &Engine::Empty)
      .def("reset", &Engine::Reset)
      .def("json_metrics", &Engine::JSONMetrics)
      .def("debug_stats", &Engine::DebugStats)
      .def("config_json", [](Engine& e) { return e.Config().AsJSON().dump(); })
      .def("set_stream_callback", [](Engine& e, py::object cb) { e.SetStreamCallback(WrapCallback(cb)); });

  py::class_<JsonFFIEngine>(m, "JsonFFIEngine")
      .def(py::init([](py::object factory, std::shared_ptr<Tokenizer> tokenizer, const std::string& conv_json,
                       const std::string& model_name, py::object callback) {
             auto holder = std::make_shared<py::object>(std::move(factory));
             ThreadedEngine::EngineFactory fn = [holder](const std::string& cfg, StreamCallback cb) {
               py::gil_scoped_acquire gil;
               py::object eng = (*holder)(cfg);
               Engine* raw = eng.cast<Engine*>();
               raw->SetStreamCallback(cb);
               return std::unique_ptr<Engine>(new ProxyEngine(std::move(eng), raw));
             };
             auto cb_holder = std::make_shared<py::object>(std::move(callback));
             JsonFFIEngine::JSONCallback cb = [cb_holder](const std::string& chunks_json) {
               py::gil_scoped_acquire gil;
               (*cb_holder)(chunks_json);
             };
             return new JsonFFIEngine(fn, std::move(tokenizer), conv_json, model_name, cb);
           }))
      .def("chat_completion", &JsonFFIEngine::ChatCompletion, py::call_guard<py::gil_scoped_release>())
      .def("set_image_embedder",
           [](JsonFFIEngine& e, py::object fn) {
             auto holder = std::make_shared<py::object>(std::move(fn));
             e.SetImageEmbedder([holder](const std::string& bytes) {
               py::gil_scoped_acquire gil;
               py::tuple r = (*holder)(py::bytes(bytes)).cast<py::tuple>();
               return std::make_pair(r[0].cast<int64_t>(), r[1].cast<int32_t>());
             });
           })
      .def_static("decode_data_url", [](const std::string& url) { return py::bytes(JsonFFIEngine::DecodeDataURL(url)); })
      .def("abort", &JsonFFIEngine::Abort, py::call_guard<py::gil_scoped_release>())
      .def("get_last_error", &JsonFFIEngine::GetLastError)
      .def("reload", &JsonFFIEngine::Reload, py::call_guard<py::gil_scoped_release>())
      .def("unload", &JsonFFIEngine::Unload, py::call_guard<py::gil_scoped_release>())
      .def("reset", &JsonFFIEngine::Reset, py::call_guard<py::gil_scoped_release>())
      .def("run_background_loop", &JsonFFIEngine::RunBackgroundLoop, py::call_guard<py::gil_scoped_release>())
      .def("run_background_stream_back_loop", &JsonFFIEngine::RunBackgroundStreamBackLoop,
           py::call_guard<py::gil_scoped_release>())
      .def("exit_background_loop", &JsonFFIEngine::ExitBackgroundLoop, py::call_guard<py::gil_scoped_release>())
      .def("json_metrics", &JsonFFIEngine::JSONMetrics);

  py::class_<ThreadedEngine>(m, "ThreadedEngine")
      .def(py::init([](py::object factory, py::object frontend_callback) {
             // factory(engine_config_json) -> _core.Engine. The Python object stays the owner; the
             // threaded engine drives it through a forwarding proxy that keeps it alive.
             auto holder = std::make_shared<py::object>(std::move(factory));
             ThreadedEngine::EngineFactory fn = [holder](const std::string& cfg, StreamCallback cb) {
               py::gil_scoped_acquire gil;
               py::object eng = (*holder)(cfg);
               Engine* raw = eng.cast<Engine*>();
               raw->SetStreamCallback(cb);
               return std::unique_ptr<Engine>(new ProxyEngine(std::move(eng), raw));
             };
             return new ThreadedEngine(fn, WrapCallback(frontend_callback));
           }))
      .def("reload", &ThreadedEngine::Reload, py::call_guard<py::gil_scoped_release>())
      .def("unload", &ThreadedEngine::Unload, py::call_guard<py::gil_scoped_release>())
      .def("reset", &ThreadedEngine::Reset, py::call_guard<py::gil_scoped_release>())
      .def("add_request",
           [](ThreadedEngine& e, const std::string& id, const py::list& inputs, const std::string& gen_cfg_json) {
             GenerationConfig g = GenerationConfig::FromJSON(gen_cfg_json, e.DefaultGenerationConfig());
             Request r = MakeRequest(id, inputs, g);
             py::gil_scoped_release rel;
             e.AddRequest(std::move(r));
           })
      .def("abort_request", &ThreadedEngine::AbortRequest, py::call_guard<py::gil_scoped_release>())
      .def("accumulate_outputs",
           [](ThreadedEngine& e, const std::string& id, int n, std::shared_ptr<Tokenizer> tok) {
             e.AccumulateOutputs(id, n, std::move(tok));
           },
           py::arg("request_id"), py::arg("num_choices"), py::arg("tokenizer"))
      .def("run_background_loop", &ThreadedEngine::RunBackgroundLoop, py::call_guard<py::gil_scoped_release>())
      .def("run_background_stream_back_loop", &ThreadedEngine::RunBackgroundStreamBackLoop,
           py::call_guard<py::gil_scoped_release>())
      .def("exit_background_loop", &ThreadedEngine::ExitBackgroundLoop, py::call_guard<py::gil_scoped_release>())
      .def("json_metrics", &ThreadedEngine::JSONMetrics)
      .def("get_complete_engine_config", &ThreadedEngine::CompleteEngineConfigJSON)
      .def("default_generation_config_json",
           [](ThreadedEngine& e) { return e.DefaultGenerationConfig().AsJSON().dump(); })
      .def("last_error", &ThreadedEngine::last_error);
}
