// The continuous-batching serving engine: requests, per-request state, scheduling actions
// (prefill with chunking / hybrid decode, batched decode, preemption, speculative draft + verify,
// grammar jump-forward), post-processing into stream outputs, and a threaded wrapper with an
// instruction queue and a stream-back loop.
//
// The model itself is behind `ModelBackend`: one call per scheduling step carries the index arrays
// built by the KV manager plus the sampling parameters, and returns the sampled tokens. Logits and
// probabilities never leave the device.
//
// Behavioural counterparts: cpp/serve/engine.cc (AddRequest :668-728, Step :749-769, abort
// :106-149, mock echo engine :160-341), cpp/serve/engine_actions/* (admission control
// batch_prefill_base.cc:51-270, decode batch_decode.cc:44-201, preemption action_commons.cc:333-427,
// post-processing action_commons.cc:177-331, draft/verify batch_draft.cc / batch_verify.cc),
// cpp/serve/request_state.cc:175-263 (finish rules) and cpp/serve/threaded_engine.cc:31-401.
#pragma once
#include <stdexcept>
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <random>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "config.h"
#include "kv_manager.h"
#include "metrics.h"
#include "prefix_cache.h"
#include "tokenizer.h"

namespace mlcb {

// ------------------------------------------------------------------ data
struct InputItem {
  // kind 0: token ids; kind 1: precomputed embedding rows held by the backend under `embed_handle`.
  int kind = 0;
  std::vector<int32_t> tokens;
  int64_t embed_handle = -1;
  int32_t embed_len = 0;
  int64_t Length() const { return kind == 0 ? static_cast<int64_t>(tokens.size()) : embed_len; }
};

struct Request {
  std::string id;
  std::vector<InputItem> inputs;
  GenerationConfig cfg;
  int64_t prompt_tokens = 0;
};

struct SampleResult {
  int32_t token = 0;
  float prob = 1.f;
  std::vector<std::pair<int32_t, float>> top;  // top-logprob candidates (token, prob)
};

struct RequestStreamOutput {
  std::string request_id;
  std::vector<std::vector<int32_t>> group_delta_token_ids;
  std::vector<std::vector<std::string>> group_delta_logprob_json_strs;
  std::vector<std::string> group_finish_reason;  // "" while running
  std::vector<std::string> group_extra_prefix_string;
  // Set on the single, merged output of a request registered with ThreadedEngine::AccumulateOutputs:
  // group_extra_prefix_string then holds each choice's complete, already detokenised text.
  bool text_is_final = false;
  std::string request_final_usage_json_str;      // non-empty on the last output of the request
};

// ------------------------------------------------------------------ backend interface
struct SampleParams {
  // one entry per sampled row
  std::vector<int32_t> logit_token_index;  // which appended token's hidden state feeds the lm head
  std::vector<float> temperature, top_p, uniform;
  std::vector<int32_t> top_k;
  std::vector<float> penalties;            // [n, 3] presence, frequency, repetition (empty: none)
  std::vector<int32_t> pen_row, pen_token, pen_count;   // appeared-token entries
  std::vector<int32_t> bias_row, bias_token;
  std::vector<float> bias_value;
  std::vector<int32_t> mask_rows;          // rows that carry a grammar bitmask
  std::vector<int32_t> mask_bits;          // [len(mask_rows), ceil(V/32)]
  int32_t num_top_logprobs = 0;            // max over rows
  // speculative decoding
  std::vector<int32_t> prob_slots;         // when non-empty: also store each row's distribution here
};

struct SampleOutput {
  std::vector<int32_t> tokens;
  std::vector<float> probs;
  std::vector<int32_t> top_tokens;  // [n, num_top_logprobs]
  std::vector<float> top_probs;
};

struct VerifyParams {
  // per sequence: its draft nodes occupy [node_indptr[i], node_indptr[i+1]) of the flat arrays.
  std::vector<int32_t> node_indptr;
  std::vector<int32_t> draft_tokens;       // token of each draft node
  std::vector<int32_t> draft_prob_slots;   // where the draft model stored each node's distribution
  std::vector<int32_t> parents;            // parent node inside the sequence's chunk, -1 = root
  std::vector<float> uniform;              // per node
  std::vector<float> final_uniform;        // per sequence, for the bonus / resampled token
  SampleParams sampling;                   // per row = per (root + node) of every sequence
  bool want_logprobs = false;              // some request reports log-probabilities: return the target's
};

struct VerifyOutput {
  std::vector<int32_t> accepted_indptr;    // per sequence
  std::vector<int32_t> accepted_nodes;     // accepted node indices (chunk-local), path order
  std::vector<int32_t> final_tokens;       // per sequence: token sampled after the accepted path
  std::vector<float> final_probs;
  // when log-probabilities are asked for: the target's probability of every accepted token (same order as
  // accepted_nodes) and, with num_top > 0, its num_top best (token, probability) pairs for every accepted token
  // followed by every final token
  std::vector<float> accepted_probs;
  std::vector<int32_t> top_tokens;
  std::vector<float> top_probs;
  int32_t num_top = 0;
};

class ModelBackend {
 public:
  virtual ~ModelBackend() = default;
  // Runs model `model_id` over the appended tokens and samples one token per SampleParams row.
  // `embed_handles[i] >= 0` replaces token i.. by backend-held embedding rows.
  virtual SampleOutput ForwardSample(int model_id, const ForwardPlan& plan,
                                     const std::vector<int32_t>& token_ids,
                                     const std::vector<int64_t>& embed_handles,
                                     const SampleParams& sampling) = 0;
  // Deferred-read form of ForwardSample for decode batches: the call returns once the work is queued.
  // `token_src[i] >= 0` says that token i is the one sampled for row token_src[i] of the previous
  // LaunchSample call on this model, which the backend still holds on the device (token_ids[i] is
  // ignored then). Returns false when the backend cannot run this step that way (nothing was done).
  virtual bool LaunchSample(int /*model_id*/, const ForwardPlan& /*plan*/, const std::vector<int32_t>& /*token_ids*/,
                            const std::vector<int32_t>& /*token_src*/, const SampleParams& /*sampling*/) {
    return false;
  }
  // Blocks for the result of the oldest LaunchSample call that has not been read yet.
  virtual SampleOutput WaitSample(int /*model_id*/) { throw std::runtime_error("no deferred sample to wait for"); }
  // Main-model pass over draft token trees followed by on-device acceptance.
  virtual VerifyOutput ForwardVerify(int model_id, const ForwardPlan& plan,
                                     const std::vector<int32_t>& token_ids,
                                     const VerifyParams& verify) = 0;
  // Applies (src_slot, dst_slot) token moves in the KV pages of `model_id` (tree commit).
  virtual void MoveKVTokens(int model_id, const std::vector<int32_t>& moves) = 0;
  // Applies (src_page, dst_page) copies outside a forward call (KV reserved for a remote sender).
  virtual void ApplyPageCopies(int /*model_id*/, const std::vector<int32_t>& /*copies*/) {
    throw std::runtime_error("this backend cannot reserve KV for disaggregated serving");
  }
  // Copies the KV entries at `src_slots` of `model_id` into the receiver described by `metadata`
  // (opaque payload produced by the receiving engine's prepare-receive step). Blocks until done.
  virtual void SendKV(int /*model_id*/, const std::vector<int32_t>& /*src_slots*/, const std::string& /*metadata*/) {
    throw std::runtime_error("this backend cannot send KV to a remote engine");
  }
  virtual void Synchronize() {}
  virtual void ReleaseEmbedding(int64_t /*handle*/) {}
  virtual void Reset() {}
};

// Grammar-constrained decoding (JSON mode). Implemented over xgrammar on the Python side.
class GrammarBackend {
 public:
  virtual ~GrammarBackend() = default;
  virtual int64_t Create(const std::string& response_format_json) = 0;
  virtual void Release(int64_t handle) = 0;
  virtual std::vector<int32_t> NextTokenBitmask(int64_t handle) = 0;
  virtual bool AcceptToken(int64_t handle, int32_t token) = 0;
  virtual void Rollback(int64_t handle, int n) = 0;
  virtual bool IsTerminated(int64_t handle) = 0;
  virtual std::string FindJumpForwardString(int64_t handle) = 0;
};

// ------------------------------------------------------------------ request state
enum class EntryStatus { kPending, kAlive, kFinished };

struct ModelState {
  int64_t internal_id = -1;                 // sequence id inside the KV manager (-1: none yet)
  std::deque<InputItem> inputs;             // not yet prefilled
  int64_t num_prefilled_tokens = 0;
  std::vector<int32_t> prefilled_tokens;    // tokens whose KV exists (fed to the prefix cache)
  int64_t cached_committed_tokens = 0;      // committed tokens already announced to the prefix cache
  // speculative decoding: chain / tree of draft tokens proposed for the next verify step
  std::vector<SampleResult> draft_tokens;
  std::vector<int32_t> draft_slots;
  std::vector<int32_t> draft_parents;
  int64_t num_tokens_for_next_decode = 0;
  int64_t jump_forward_inputs = 0;          // pending inputs that are grammar-forced output tokens
};

struct RequestStateEntry {
  EntryStatus status = EntryStatus::kPending;
  int parent_idx = -1;
  std::vector<int> child_indices;
  std::vector<ModelState> mstates;          // one per model (main, draft)
  std::vector<SampleResult> committed_tokens;
  std::unordered_map<int32_t, int32_t> appeared_token_ids;
  std::unique_ptr<StopStrHandler> stop_handler;
  std::mt19937_64 rng;
  int64_t next_callback_token_pos = 0;      // committed tokens already handed to the stop handler
  int64_t logprob_cursor = 0;               // committed tokens whose logprob entry was emitted
  int64_t grammar_handle = -1;
  std::string finish_reason;
  std::string extra_prefix_string;
  bool kv_released = false;
  int inflight_row = -1;                    // row of this entry in the decode step whose result is not read yet
  double NextUniform() { return std::uniform_real_distribution<double>(0.0, 1.0)(rng); }
};

struct RequestState {
  Request request;
  std::vector<RequestStateEntry> entries;   // [0] = root; children follow when n > 1
  RequestMetrics metrics;
  bool prefill_done = false;
  int num_unfinished = 0;
  // disaggregated serving: KV for positions [.., disagg_reserved_end) is reserved / being received
  // and the request waits for its start-generation step (-1: not such a request)
  int64_t disagg_reserved_end = -1;
  int64_t disagg_matched = 0;
};

// ------------------------------------------------------------------ engine
using StreamCallback = std::function<void(std::vector<RequestStreamOutput>)>;

struct EngineModelInfo {
  int64_t vocab_size = 0;
  int64_t num_pages = 0;
  std::vector<int32_t> eos_token_ids;
  std::string generation_defaults_json;     // the model's mlc-chat-config.json
};

class Engine {
 public:
  virtual ~Engine() = default;
  virtual void AddRequest(Request request) = 0;
  virtual void AbortRequest(const std::string& request_id) = 0;
  virtual void AbortAllRequests() = 0;
  virtual void Step() = 0;
  virtual bool Empty() const = 0;
  virtual void Reset() = 0;
  virtual std::string JSONMetrics() const = 0;
  virtual const GenerationConfig& DefaultGenerationConfig() const = 0;
  virtual const EngineConfig& Config() const = 0;
  virtual void SetStreamCallback(StreamCallback cb) = 0;
  // Step-level statistics for tests (number of prefill / decode steps taken, preemptions).
  virtual std::string DebugStats() const { return "{}"; }

  static std::unique_ptr<Engine> Create(EngineConfig config, std::vector<EngineModelInfo> models,
                                        std::shared_ptr<ModelBackend> backend,
                                        std::shared_ptr<const Tokenizer> tokenizer,
                                        std::shared_ptr<GrammarBackend> grammar,
                                        std::shared_ptr<EventTraceRecorder> trace,
                                        StreamCallback callback);
  // Echo engine behind model_lib == "mock://echo": streams the prompt tokens back and reports the
  // parsed generation config in usage.extra.
  static std::unique_ptr<Engine> CreateMockEcho(EngineConfig config, std::string model_config_json,
                                                std::shared_ptr<const Tokenizer> tokenizer,
                                                StreamCallback callback);
};

// ------------------------------------------------------------------ threaded engine
class ThreadedEngine {
 public:
  using EngineFactory = std::function<std::unique_ptr<Engine>(const std::string& engine_config_json,
                                                              StreamCallback callback)>;
  ThreadedEngine(EngineFactory factory, StreamCallback frontend_callback);
  ~ThreadedEngine();

  void Reload(const std::string& engine_config_json);  // blocks until the engine is rebuilt
  void Unload();                                        // blocks
  void Reset();                                         // blocks
  void AddRequest(Request request);
  void AbortRequest(const std::string& request_id);
  // Non-streaming consumers: keep this request's per-step outputs in the stream-back thread (tokens,
  // logprobs, detokenised text) and hand the frontend one merged output when the request is done,
  // instead of one callback per request and step. Call before AddRequest.
  void AccumulateOutputs(const std::string& request_id, int num_choices, std::shared_ptr<const Tokenizer> tokenizer);
  void RunBackgroundLoop();             // call on a dedicated thread
  void RunBackgroundStreamBackLoop();   // call on a dedicated thread
  void ExitBackgroundLoop();
  std::string JSONMetrics();
  std::string CompleteEngineConfigJSON();
  GenerationConfig DefaultGenerationConfig();
  std::string last_error();

 private:
  enum class Kind { kAddRequest, kAbortRequest, kUnload, kReload, kReset, kDebugCall };
  struct Instruction {
    Kind kind;
    std::shared_ptr<Request> request;
    std::string arg;
  };
  void HandleReload(const std::string& cfg);
  void HandleUnload();

  EngineFactory factory_;
  StreamCallback frontend_callback_;
  std::unique_ptr<Engine> engine_;
  std::mutex engine_mu_;  // guards engine_ for metric / config queries from other threads

  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<Instruction> queue_;
  std::atomic<bool> exit_{false};
  std::atomic<bool> engine_waiting_{false};

  std::mutex reload_mu_;
  std::condition_variable reload_cv_;
  bool reload_done_ = false, unload_done_ = false, reset_done_ = false;
  std::string error_;

  std::mutex sb_mu_;
  std::condition_variable sb_cv_;
  std::vector<RequestStreamOutput> sb_queue_;
  std::atomic<bool> sb_waiting_{false};
  struct OutputAccumulator {
    RequestStreamOutput merged;
    std::vector<TextStreamer> streamers;
    std::vector<bool> finished;
  };
  std::mutex acc_mu_;
  std::unordered_map<std::string, OutputAccumulator> acc_;
  // Folds `out` into its request's accumulator. Returns true when `out` should go to the frontend (it
  // was not an accumulated request, or it now carries the merged, final result).
  bool Accumulate(RequestStreamOutput* out);
  std::atomic<int64_t> pending_outputs_{0};
};

}  // namespace mlcb
