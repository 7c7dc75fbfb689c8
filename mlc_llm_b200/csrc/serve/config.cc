#include "config.h"

#include <algorithm>
#include <cmath>
#include <sstream>
#include <stdexcept>

namespace mlcb {

using json::Object;
using json::Value;

std::string ToString(EngineMode m) {
  return m == EngineMode::kLocal ? "local" : m == EngineMode::kInteractive ? "interactive" : "server";
}
std::string ToString(SpeculativeMode m) {
  switch (m) {
    case SpeculativeMode::kSmallDraft: return "small_draft";
    case SpeculativeMode::kEagle: return "eagle";
    case SpeculativeMode::kMedusa: return "medusa";
    default: return "disable";
  }
}
std::string ToString(PrefixCacheMode m) { return m == PrefixCacheMode::kRadix ? "radix" : "disable"; }
std::string ToString(PrefillMode m) { return m == PrefillMode::kHybrid ? "hybrid" : "chunked"; }

// ------------------------------------------------------------------ ResponseFormat / Debug
Value ResponseFormat::AsJSON() const {
  Object o;
  o["type"] = type;
  if (schema.has_value()) o["schema"] = *schema;
  return Value(std::move(o));
}

Value DisaggConfig::AsJSON() const {
  Object o;
  switch (kind) {
    case DisaggRequestKind::kPrepareReceive: o["kind"] = "prepare_receive"; break;
    case DisaggRequestKind::kRemoteSend: o["kind"] = "remote_send"; break;
    case DisaggRequestKind::kStartGeneration: o["kind"] = "start_generation"; break;
    default: break;
  }
  if (!kv_append_metadata.empty()) o["kv_append_metadata"] = kv_append_metadata;
  if (kv_window_begin) o["kv_window_begin"] = *kv_window_begin;
  if (kv_window_end) o["kv_window_end"] = *kv_window_end;
  if (dst_group_offset) o["dst_group_offset"] = *dst_group_offset;
  return Value(std::move(o));
}

DebugConfig DebugConfig::FromJSON(const Object& o) {
  DebugConfig d;
  d.ignore_eos = json::get_or<bool>(o, "ignore_eos", false);
  d.pinned_system_prompt = json::get_or<bool>(o, "pinned_system_prompt", false);
  std::string sr = json::get_or<std::string>(o, "special_request", "");
  if (sr == "query_engine_metrics") d.special_request = SpecialRequestKind::kQueryEngineMetrics;
  else if (!sr.empty()) throw std::runtime_error("Unknown special request " + sr);
  std::string gm = json::get_or<std::string>(o, "grammar_execution_mode", "jump_forward");
  if (gm == "jump_forward") d.grammar_execution_mode = GrammarExecutionMode::kJumpForward;
  else if (gm == "constraint") d.grammar_execution_mode = GrammarExecutionMode::kConstraint;
  else throw std::runtime_error("Unknown grammar execution mode " + gm);
  if (auto* dc = o.find("disagg_config"); dc && dc->is_object()) {
    const Object& c = dc->as_object();
    std::string kind = json::get_or<std::string>(c, "kind", "");
    if (kind == "prepare_receive") d.disagg_config.kind = DisaggRequestKind::kPrepareReceive;
    else if (kind == "remote_send") d.disagg_config.kind = DisaggRequestKind::kRemoteSend;
    else if (kind == "start_generation") d.disagg_config.kind = DisaggRequestKind::kStartGeneration;
    else if (!kind.empty()) throw std::runtime_error("Unknown disaggregation request kind " + kind);
    d.disagg_config.kv_append_metadata = json::get_or<std::string>(c, "kv_append_metadata", "");
    if (auto* v = c.find("kv_window_begin"); v && v->is_number()) d.disagg_config.kv_window_begin = v->as_int();
    if (auto* v = c.find("kv_window_end"); v && v->is_number()) d.disagg_config.kv_window_end = v->as_int();
    if (auto* v = c.find("dst_group_offset"); v && v->is_number()) d.disagg_config.dst_group_offset = v->as_int();
  }
  return d;
}

Value DebugConfig::AsJSON() const {
  Object o;
  o["ignore_eos"] = ignore_eos;
  o["pinned_system_prompt"] = pinned_system_prompt;
  if (special_request == SpecialRequestKind::kQueryEngineMetrics)
    o["special_request"] = "query_engine_metrics";
  o["grammar_execution_mode"] =
      grammar_execution_mode == GrammarExecutionMode::kJumpForward ? "jump_forward" : "constraint";
  if (disagg_config.kind != DisaggRequestKind::kNone) o["disagg_config"] = disagg_config.AsJSON();
  return Value(std::move(o));
}

// ------------------------------------------------------------------ GenerationConfig
GenerationConfig GenerationConfig::DefaultsFromModelConfig(const Object& c) {
  GenerationConfig g;
  g.temperature = json::get_or<double>(c, "temperature", 1.0);
  g.top_p = json::get_or<double>(c, "top_p", 1.0);
  g.frequency_penalty = json::get_or<double>(c, "frequency_penalty", 0.0);
  g.presence_penalty = json::get_or<double>(c, "presence_penalty", 0.0);
  g.repetition_penalty = json::get_or<double>(c, "repetition_penalty", 1.0);
  return g;
}

GenerationConfig GenerationConfig::FromJSON(const std::string& json_str, const GenerationConfig& dflt) {
  Value root = json::parse(json_str);
  if (!root.is_object()) throw std::runtime_error("generation config must be a JSON object");
  const Object& o = root.as_object();
  GenerationConfig g = dflt;
  g.n = json::get_or<int>(o, "n", 1);
  if (g.n <= 0) throw std::runtime_error("\"n\" should be at least 1");
  g.temperature = json::get_or<double>(o, "temperature", dflt.temperature);
  if (g.temperature < 0) throw std::runtime_error("\"temperature\" should be non-negative");
  g.top_p = json::get_or<double>(o, "top_p", dflt.top_p);
  if (g.top_p < 0 || g.top_p > 1) throw std::runtime_error("\"top_p\" should be in range [0, 1]");
  g.top_k = json::get_or<int>(o, "top_k", 0);
  g.frequency_penalty = json::get_or<double>(o, "frequency_penalty", dflt.frequency_penalty);
  if (std::fabs(g.frequency_penalty) > 2.0) throw std::runtime_error("frequency penalty must be in [-2, 2]");
  g.presence_penalty = json::get_or<double>(o, "presence_penalty", dflt.presence_penalty);
  if (std::fabs(g.presence_penalty) > 2.0) throw std::runtime_error("presence penalty must be in [-2, 2]");
  g.repetition_penalty = json::get_or<double>(o, "repetition_penalty", dflt.repetition_penalty);
  if (g.repetition_penalty <= 0) throw std::runtime_error("\"repetition_penalty\" must be positive");
  g.logprobs = json::get_or<bool>(o, "logprobs", false);
  g.top_logprobs = json::get_or<int>(o, "top_logprobs", 0);
  if (g.top_logprobs < 0 || g.top_logprobs > 20)
    throw std::runtime_error("At most 20 top logprob tokens are supported");
  if (g.top_logprobs != 0 && !g.logprobs)
    throw std::runtime_error("\"logprobs\" must be true to support \"top_logprobs\"");
  g.logit_bias.clear();
  if (auto* lb = o.find("logit_bias"); lb && lb->is_object()) {
    for (auto& m : lb->as_object().members()) {
      double b = m.second.as_double();
      if (std::fabs(b) > 100.0) throw std::runtime_error("Logit bias value should be in range [-100, 100].");
      g.logit_bias.emplace_back(std::stoi(m.first), static_cast<float>(b));
    }
  }
  if (auto* v = o.find("seed"); v && v->is_number()) g.seed = v->as_int();
  if (auto* v = o.find("max_tokens"); v && v->is_number()) g.max_tokens = v->as_int();
  g.stop_strs.clear();
  if (auto* v = o.find("stop_strs"); v && v->is_array())
    for (auto& s : v->as_array()) g.stop_strs.push_back(s.as_string());
  g.stop_token_ids.clear();
  if (auto* v = o.find("stop_token_ids"); v && v->is_array())
    for (auto& s : v->as_array()) g.stop_token_ids.push_back(static_cast<int>(s.as_int()));
  if (auto* v = o.find("response_format"); v && v->is_object()) {
    const Object& rf = v->as_object();
    g.response_format.type = json::get_or<std::string>(rf, "type", "text");
    if (g.response_format.type != "text" && g.response_format.type != "json_object")
      throw std::runtime_error("Unknown response_format type " + g.response_format.type);
    if (auto* sc = rf.find("schema"); sc && sc->is_string()) g.response_format.schema = sc->as_string();
  }
  if (auto* v = o.find("debug_config"); v && v->is_object()) g.debug_config = DebugConfig::FromJSON(v->as_object());
  return g;
}

Value GenerationConfig::AsJSON() const {
  Object o;
  o["n"] = n;
  o["temperature"] = temperature;
  o["top_p"] = top_p;
  if (top_k > 0) o["top_k"] = top_k;
  o["frequency_penalty"] = frequency_penalty;
  o["presence_penalty"] = presence_penalty;
  o["repetition_penalty"] = repetition_penalty;
  o["logprobs"] = logprobs;
  o["top_logprobs"] = top_logprobs;
  Object lb;
  for (auto& p : logit_bias) lb[std::to_string(p.first)] = static_cast<double>(p.second);
  o["logit_bias"] = Value(std::move(lb));
  o["seed"] = seed;
  o["max_tokens"] = max_tokens;
  json::Array ss;
  for (auto& s : stop_strs) ss.emplace_back(s);
  o["stop_strs"] = Value(std::move(ss));
  json::Array st;
  for (int t : stop_token_ids) st.emplace_back(t);
  o["stop_token_ids"] = Value(std::move(st));
  o["response_format"] = response_format.AsJSON();
  o["debug_config"] = debug_config.AsJSON();
  return Value(std::move(o));
}

// ------------------------------------------------------------------ EngineConfig
static int64_t opt_int(const Object& o, const char* k) {
  auto* v = o.find(k);
  return (v && v->is_number()) ? v->as_int() : -1;
}

EngineConfig EngineConfig::FromJSON(const std::string& json_str) {
  Value root = json::parse(json_str);
  const Object& o = root.as_object();
  EngineConfig c;
  c.model = json::get_or<std::string>(o, "model", "");
  c.model_lib = json::get_or<std::string>(o, "model_lib", "");
  if (auto* am = o.find("additional_models"); am && am->is_array()) {
    for (auto& e : am->as_array()) {
      if (e.is_string()) c.additional_models.emplace_back(e.as_string(), "");
      else if (e.is_array() && !e.as_array().empty())
        c.additional_models.emplace_back(
            e.as_array()[0].as_string(),
            e.as_array().size() > 1 && e.as_array()[1].is_string() ? e.as_array()[1].as_string() : "");
    }
  }
  std::string mode = json::get_or<std::string>(o, "mode", "local");
  if (mode == "local") c.mode = EngineMode::kLocal;
  else if (mode == "interactive") c.mode = EngineMode::kInteractive;
  else if (mode == "server") c.mode = EngineMode::kServer;
  else throw std::runtime_error("Invalid engine mode " + mode);
  c.tensor_parallel_shards = std::max<int>(1, json::get_or<int>(o, "tensor_parallel_shards", 1));
  c.pipeline_parallel_stages = std::max<int>(1, json::get_or<int>(o, "pipeline_parallel_stages", 1));
  c.opt = json::get_or<std::string>(o, "opt", "");
  c.gpu_memory_utilization = json::get_or<double>(o, "gpu_memory_utilization", 0.85);
  if (c.gpu_memory_utilization <= 0 || c.gpu_memory_utilization > 1)
    throw std::runtime_error("gpu_memory_utilization must be in (0, 1]");
  c.kv_cache_page_size = json::get_or<int>(o, "kv_cache_page_size", 16);
  if (c.kv_cache_page_size != 16) throw std::runtime_error("KV cache page size other than 16 is not supported.");
  c.max_num_sequence = opt_int(o, "max_num_sequence");
  c.max_total_sequence_length = opt_int(o, "max_total_sequence_length");
  c.max_single_sequence_length = opt_int(o, "max_single_sequence_length");
  c.prefill_chunk_size = opt_int(o, "prefill_chunk_size");
  c.sliding_window_size = opt_int(o, "sliding_window_size");
  c.attention_sink_size = opt_int(o, "attention_sink_size");
  c.max_history_size = opt_int(o, "max_history_size");
  c.kv_state_kind = json::get_or<std::string>(o, "kv_state_kind", "kv_cache");
  std::string sm = json::get_or<std::string>(o, "speculative_mode", "disable");
  if (sm == "disable") c.speculative_mode = SpeculativeMode::kDisable;
  else if (sm == "small_draft") c.speculative_mode = SpeculativeMode::kSmallDraft;
  else if (sm == "eagle") c.speculative_mode = SpeculativeMode::kEagle;
  else if (sm == "medusa") c.speculative_mode = SpeculativeMode::kMedusa;
  else throw std::runtime_error("Invalid speculative mode " + sm);
  c.spec_draft_length = json::get_or<int>(o, "spec_draft_length", 0);
  c.spec_tree_width = json::get_or<int>(o, "spec_tree_width", 1);
  std::string pm = json::get_or<std::string>(o, "prefix_cache_mode", "radix");
  if (pm == "radix") c.prefix_cache_mode = PrefixCacheMode::kRadix;
  else if (pm == "disable") c.prefix_cache_mode = PrefixCacheMode::kDisable;
  else throw std::runtime_error("Invalid prefix cache mode " + pm);
  c.prefix_cache_max_num_recycling_seqs = opt_int(o, "prefix_cache_max_num_recycling_seqs");
  std::string fm = json::get_or<std::string>(o, "prefill_mode", "hybrid");
  if (fm == "hybrid") c.prefill_mode = PrefillMode::kHybrid;
  else if (fm == "chunked") c.prefill_mode = PrefillMode::kChunked;
  else throw std::runtime_error("Invalid prefill mode " + fm);
  c.verbose = json::get_or<bool>(o, "verbose", true);
  return c;
}

Value EngineConfig::AsJSON() const {
  Object o;
  o["model"] = model;
  o["model_lib"] = model_lib;
  json::Array am;
  for (auto& p : additional_models) {
    json::Array pair;
    pair.emplace_back(p.first);
    pair.emplace_back(p.second);
    am.emplace_back(std::move(pair));
  }
  o["additional_models"] = Value(std::move(am));
  o["mode"] = ToString(mode);
  o["tensor_parallel_shards"] = tensor_parallel_shards;
  o["pipeline_parallel_stages"] = pipeline_parallel_stages;
  o["opt"] = opt;
  o["gpu_memory_utilization"] = gpu_memory_utilization;
  o["kv_cache_page_size"] = kv_cache_page_size;
  o["max_num_sequence"] = max_num_sequence;
  o["max_total_sequence_length"] = max_total_sequence_length;
  o["max_single_sequence_length"] = max_single_sequence_length;
  o["prefill_chunk_size"] = prefill_chunk_size;
  o["sliding_window_size"] = sliding_window_size;
  o["attention_sink_size"] = attention_sink_size;
  o["max_history_size"] = max_history_size;
  o["kv_state_kind"] = kv_state_kind;
  o["speculative_mode"] = ToString(speculative_mode);
  o["spec_draft_length"] = spec_draft_length;
  o["spec_tree_width"] = spec_tree_width;
  o["prefix_cache_mode"] = ToString(prefix_cache_mode);
  o["prefix_cache_max_num_recycling_seqs"] = prefix_cache_max_num_recycling_seqs;
  o["prefill_mode"] = ToString(prefill_mode);
  o["verbose"] = verbose;
  return Value(std::move(o));
}

// ------------------------------------------------------------------ capacity inference
CapacityResult InferCapacity(const EngineConfig& user, const std::vector<ModelCapacityInfo>& models,
                             int64_t gpu_total_bytes) {
  if (models.empty()) throw std::runtime_error("InferCapacity: no model");
  CapacityResult res;
  EngineConfig c = user;
  const ModelCapacityInfo& m0 = models[0];
  // model-imposed limits
  int64_t model_max_single = INT64_MAX, model_prefill_chunk = INT64_MAX, model_max_batch = INT64_MAX;
  for (auto& m : models) {
    int64_t single = m.context_window_size > 0 ? m.context_window_size : INT64_MAX;
    model_max_single = std::min(model_max_single, single);
    model_prefill_chunk = std::min(model_prefill_chunk, m.prefill_chunk_size);
    model_max_batch = std::min(model_max_batch, m.max_batch_size);
  }
  if (c.sliding_window_size < 0 && m0.sliding_window_size > 0 && m0.context_window_size <= 0)
    c.sliding_window_size = m0.sliding_window_size;
  const bool windowed = c.sliding_window_size > 0;
  if (windowed && c.attention_sink_size < 0) c.attention_sink_size = 0;

  // 1. batch size by mode
  if (c.max_num_sequence <= 0) {
    switch (c.mode) {
      case EngineMode::kLocal: c.max_num_sequence = std::min<int64_t>(4, model_max_batch); break;
      case EngineMode::kInteractive: c.max_num_sequence = 1; break;
      case EngineMode::kServer: c.max_num_sequence = model_max_batch; break;
    }
  }
  // 2. single-sequence limit
  if (c.max_single_sequence_length <= 0)
    c.max_single_sequence_length = model_max_single == INT64_MAX ? (1 << 30) : model_max_single;
  else if (model_max_single != INT64_MAX)
    c.max_single_sequence_length = std::min(c.max_single_sequence_length, model_max_single);
  // 3. prefill chunk
  if (c.prefill_chunk_size <= 0) {
    c.prefill_chunk_size = model_prefill_chunk;
    if (windowed) c.prefill_chunk_size = std::min(c.prefill_chunk_size, c.sliding_window_size);
  }
  // 4. memory-bound total sequence length
  double kv_bytes_per_token = 0, aux = 0, workspace = 0, logit_ws = 0, params = 0;
  for (auto& m : models) {
    const int64_t layers = m.num_layers / std::max(1, m.pipeline_parallel_stages);
    kv_bytes_per_token += static_cast<double>(m.head_dim * m.num_kv_heads * layers * 2 * m.kv_bytes_per_element) + 1.25;
    const int64_t hidden = m.head_dim * m.num_qo_heads;
    aux += (c.max_num_sequence + 1) * 88.0 + c.prefill_chunk_size * (m.num_qo_heads + 1) * 8.0 +
           c.prefill_chunk_size * m.head_dim * (m.num_qo_heads + m.num_kv_heads) * 4.0 + 48.0 * 1024 * 1024;
    workspace += c.prefill_chunk_size * 4.0 + c.max_num_sequence * 4.0 +
                 (c.prefill_chunk_size * 2.0 + c.max_num_sequence) * hidden * 2.0 * 8.0;
    logit_ws += c.max_num_sequence * 20.0 + c.max_num_sequence * m.vocab_size * 16.125;
    params += static_cast<double>(m.params_bytes);
  }
  const double budget = gpu_total_bytes * c.gpu_memory_utilization - params - aux - workspace - logit_ws;
  int64_t mem_max_total = static_cast<int64_t>(budget / kv_bytes_per_token);
  std::ostringstream rep;
  rep << "memory plan: total " << gpu_total_bytes / (1 << 20) << " MB x " << c.gpu_memory_utilization
      << ", params " << static_cast<int64_t>(params) / (1 << 20) << " MB, workspace "
      << static_cast<int64_t>(aux + workspace + logit_ws) / (1 << 20) << " MB, KV "
      << kv_bytes_per_token << " B/token -> at most " << mem_max_total << " tokens";
  if (mem_max_total <= 0)
    throw std::runtime_error("Insufficient GPU memory for the KV cache: " + rep.str());
  if (c.max_total_sequence_length <= 0) {
    switch (c.mode) {
      case EngineMode::kLocal:
        c.max_total_sequence_length = std::min<int64_t>(
            {mem_max_total, c.max_single_sequence_length, int64_t(8192)});
        if (windowed) c.max_total_sequence_length = std::min<int64_t>(mem_max_total, c.max_num_sequence * c.sliding_window_size);
        break;
      case EngineMode::kInteractive:
        c.max_total_sequence_length = std::min<int64_t>(mem_max_total, c.max_single_sequence_length);
        if (windowed) c.max_total_sequence_length = std::min<int64_t>(mem_max_total, c.sliding_window_size);
        break;
      case EngineMode::kServer:
        c.max_total_sequence_length = mem_max_total;
        break;
    }
  } else if (c.max_total_sequence_length > mem_max_total) {
    throw std::runtime_error("max_total_sequence_length " + std::to_string(c.max_total_sequence_length) +
                             " exceeds what fits in memory (" + std::to_string(mem_max_total) + ")");
  }
  c.max_single_sequence_length = std::min(c.max_single_sequence_length, c.max_total_sequence_length);
  if (!windowed) c.prefill_chunk_size = std::min(c.prefill_chunk_size, c.max_total_sequence_length);
  if (c.prefix_cache_max_num_recycling_seqs < 0)
    c.prefix_cache_max_num_recycling_seqs = c.max_num_sequence;
  res.kv_bytes_per_token = kv_bytes_per_token;
  // every live or recycled sequence may waste up to one page, plus one spare for copy-on-write
  res.num_pages = (c.max_total_sequence_length + c.kv_cache_page_size - 1) / c.kv_cache_page_size +
                  2 * (c.max_num_sequence + c.prefix_cache_max_num_recycling_seqs) + 1;
  res.config = c;
  res.report = rep.str();
  return res;
}

CapacityResult InferRNNStateCapacity(const EngineConfig& user, const std::vector<ModelCapacityInfo>& models,
                                     int64_t gpu_total_bytes) {
  if (models.empty()) throw std::runtime_error("InferRNNStateCapacity: no model");
  if (user.max_single_sequence_length > 0)
    throw std::runtime_error("a recurrent state has no per-sequence length limit: max_single_sequence_length (" +
                             std::to_string(user.max_single_sequence_length) + ") must not be set");
  CapacityResult res;
  EngineConfig c = user;
  int64_t model_prefill_chunk = INT64_MAX, model_max_batch = INT64_MAX;
  for (auto& m : models) {
    model_prefill_chunk = std::min(model_prefill_chunk, m.prefill_chunk_size);
    model_max_batch = std::min(model_max_batch, m.max_batch_size);
  }
  if (c.prefill_chunk_size <= 0) c.prefill_chunk_size = std::min<int64_t>(model_prefill_chunk, 4096);
  if (c.max_num_sequence <= 0)
    c.max_num_sequence = c.mode == EngineMode::kInteractive ? 1 : std::min<int64_t>(4, model_max_batch);
  if (c.max_total_sequence_length <= 0) c.max_total_sequence_length = 32768;
  double state_per_snapshot = 0, workspace = 0, logit_ws = 0, params = 0;
  for (auto& m : models) {
    if (m.rnn_state_bytes_per_sequence <= 0)
      throw std::runtime_error("InferRNNStateCapacity: the model reports no recurrent state size");
    state_per_snapshot += static_cast<double>(c.max_num_sequence) * m.rnn_state_bytes_per_sequence;
    const int64_t hidden = m.hidden_size > 0 ? m.hidden_size : m.head_dim * m.num_qo_heads;
    workspace += c.prefill_chunk_size * 4.0 + c.max_num_sequence * 4.0 +
                 (c.prefill_chunk_size * 2.0 + c.max_num_sequence) * hidden * 2.0;
    logit_ws += c.max_num_sequence * 20.0 + c.max_num_sequence * m.vocab_size * 16.125;
    params += static_cast<double>(m.params_bytes);
  }
  const double budget = gpu_total_bytes * c.gpu_memory_utilization - params - workspace - logit_ws;
  const int64_t fit = static_cast<int64_t>(budget / state_per_snapshot);
  std::ostringstream rep;
  rep << "memory plan (recurrent state): total " << gpu_total_bytes / (1 << 20) << " MB x "
      << c.gpu_memory_utilization << ", params " << static_cast<int64_t>(params) / (1 << 20) << " MB, workspace "
      << static_cast<int64_t>(workspace + logit_ws) / (1 << 20) << " MB, state "
      << static_cast<int64_t>(state_per_snapshot) / (1 << 10) << " KB per snapshot of " << c.max_num_sequence
      << " sequences -> at most " << fit << " snapshots";
  if (fit <= 0)
    throw std::runtime_error("Insufficient GPU memory for the recurrent state: " + rep.str() +
                             "; quantise the weights or lower the prefill chunk size");
  c.max_history_size = c.max_history_size > 0 ? std::min(c.max_history_size, fit) : fit;
  c.max_single_sequence_length = c.max_total_sequence_length;
  if (c.prefix_cache_max_num_recycling_seqs < 0) c.prefix_cache_max_num_recycling_seqs = 0;
  // the engine still hands out token slots page by page (positions only; no KV memory stands behind them)
  res.num_pages = (c.max_total_sequence_length + c.kv_cache_page_size - 1) / c.kv_cache_page_size +
                  2 * c.max_num_sequence + 1;
  res.kv_bytes_per_token = 0;
  res.config = c;
  res.report = rep.str();
  return res;
}

}  // namespace mlcb
