// Engine, generation and debug configuration: JSON parsing, validation, serialisation, and the
// inference of batch / KV-cache capacity from the memory budget.
//
// Behavioural counterpart: cpp/serve/config.h:38-324 and cpp/serve/config.cc (validation bounds
// :171-202,237-267; mode presets and the KV capacity formula :688-727).
#pragma once
#include <cstdint>
#include <optional>
#include <string>
#include <utility>
#include <vector>

#include "json.h"

namespace mlcb {

enum class EngineMode { kLocal, kInteractive, kServer };
enum class PrefixCacheMode { kDisable, kRadix };
enum class SpeculativeMode { kDisable, kSmallDraft, kEagle, kMedusa };
enum class PrefillMode { kChunked, kHybrid };
enum class DisaggRequestKind { kNone, kPrepareReceive, kRemoteSend, kStartGeneration };
enum class SpecialRequestKind { kNone, kQueryEngineMetrics };
enum class GrammarExecutionMode { kConstraint, kJumpForward };

struct ResponseFormat {
  std::string type = "text";  // "text" | "json_object"
  std::optional<std::string> schema;
  json::Value AsJSON() const;
};

struct DisaggConfig {
  DisaggRequestKind kind = DisaggRequestKind::kNone;
  std::string kv_append_metadata;  // base64 payload, opaque to the config layer
  std::optional<int64_t> kv_window_begin, kv_window_end, dst_group_offset;
  json::Value AsJSON() const;
};

struct DebugConfig {
  bool ignore_eos = false;
  bool pinned_system_prompt = false;
  SpecialRequestKind special_request = SpecialRequestKind::kNone;
  GrammarExecutionMode grammar_execution_mode = GrammarExecutionMode::kJumpForward;
  DisaggConfig disagg_config;
  static DebugConfig FromJSON(const json::Object& o);
  json::Value AsJSON() const;
};

struct GenerationConfig {
  int n = 1;
  double temperature = 1.0;
  double top_p = 1.0;
  int top_k = 0;  // extension: 0 disables
  double frequency_penalty = 0.0;
  double presence_penalty = 0.0;
  double repetition_penalty = 1.0;
  bool logprobs = false;
  int top_logprobs = 0;
  std::vector<std::pair<int, float>> logit_bias;
  int64_t seed = -1;       // < 0: draw from the engine's generator
  int64_t max_tokens = -1;  // < 0: until the context window ends
  std::vector<std::string> stop_strs;
  std::vector<int> stop_token_ids;
  ResponseFormat response_format;
  DebugConfig debug_config;

  // Parses a request-level JSON on top of `defaults` (the model's mlc-chat-config values).
  // Throws std::runtime_error with a readable message on invalid values.
  static GenerationConfig FromJSON(const std::string& json_str, const GenerationConfig& defaults);
  static GenerationConfig DefaultsFromModelConfig(const json::Object& mlc_chat_config);
  json::Value AsJSON() const;
};

struct EngineConfig {
  std::string model;
  std::string model_lib;
  std::vector<std::pair<std::string, std::string>> additional_models;
  EngineMode mode = EngineMode::kLocal;
  int tensor_parallel_shards = 1;
  int pipeline_parallel_stages = 1;
  std::string opt;
  double gpu_memory_utilization = 0.85;
  int kv_cache_page_size = 16;
  int64_t max_num_sequence = -1;
  int64_t max_total_sequence_length = -1;
  int64_t max_single_sequence_length = -1;
  int64_t prefill_chunk_size = -1;
  int64_t sliding_window_size = -1;
  int64_t attention_sink_size = -1;
  int64_t max_history_size = -1;
  std::string kv_state_kind = "kv_cache";
  SpeculativeMode speculative_mode = SpeculativeMode::kDisable;
  int spec_draft_length = 0;
  int spec_tree_width = 1;
  PrefixCacheMode prefix_cache_mode = PrefixCacheMode::kRadix;
  int64_t prefix_cache_max_num_recycling_seqs = -1;
  PrefillMode prefill_mode = PrefillMode::kHybrid;
  bool verbose = true;

  static EngineConfig FromJSON(const std::string& json_str);
  json::Value AsJSON() const;
};

// What the capacity inference needs to know about one model.
struct ModelCapacityInfo {
  int64_t params_bytes = 0;         // per GPU
  int64_t num_layers = 0;
  int64_t num_qo_heads = 0;         // per GPU (after tensor parallel)
  int64_t num_kv_heads = 0;         // per GPU
  int64_t head_dim = 0;
  int64_t vocab_size = 0;
  int64_t context_window_size = -1;
  int64_t sliding_window_size = -1;
  int64_t prefill_chunk_size = 2048;
  int64_t max_batch_size = 128;
  int pipeline_parallel_stages = 1;
  int kv_bytes_per_element = 2;
  // recurrent-state models: bytes of state one sequence holds (all layers), and the hidden size that the
  // workspace estimate needs (these models have no attention heads to derive it from)
  int64_t rnn_state_bytes_per_sequence = 0;
  int64_t hidden_size = 0;
};

struct CapacityResult {
  EngineConfig config;
  int64_t num_pages = 0;
  double kv_bytes_per_token = 0;
  std::string report;
};

// Recurrent-state models (kv_state_kind "rnn_state"): no KV pages; the batch size and how many state
// snapshots per sequence (`max_history_size`) fit beside the weights. Counterpart of the reference's
// InferrableEngineConfig::InferForRNNState (cpp/serve/config.cc:903-1060): a user-set
// max_single_sequence_length is an error, the prefill chunk defaults to min(model, 4096), the batch size
// to 1 (interactive) or min(4, model), the token capacity to 32768, and max_history_size to what the memory
// left after weights and workspaces holds (at least one snapshot per sequence, or the call fails).
CapacityResult InferRNNStateCapacity(const EngineConfig& user, const std::vector<ModelCapacityInfo>& models,
                                     int64_t gpu_total_bytes);

// Fills max_num_sequence / max_total_sequence_length / max_single_sequence_length /
// prefill_chunk_size for the configured mode given `gpu_total_bytes` of device memory.
CapacityResult InferCapacity(const EngineConfig& user, const std::vector<ModelCapacityInfo>& models,
                             int64_t gpu_total_bytes);

std::string ToString(EngineMode m);
std::string ToString(SpeculativeMode m);
std::string ToString(PrefixCacheMode m);
std::string ToString(PrefillMode m);

}  // namespace mlcb
