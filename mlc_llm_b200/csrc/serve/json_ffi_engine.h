// JSON-in / JSON-out engine front end: takes OpenAI chat-completion request bodies as JSON strings,
// renders the conversation template, tokenises, drives the threaded engine, detokenises the
// stream and hands back ChatCompletionStreamResponse objects as JSON (used by the chat REPL and by
// embedders that cannot link the Python protocol layer).
//
// Behavioural counterpart: cpp/json_ffi/json_ffi_engine.{h,cc} (chat_completion / abort / reload /
// unload / reset / background loops; error string in GetLastError).
#pragma once
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "engine.h"
#include "tokenizer.h"

namespace mlcb {

class JsonFFIEngine {
 public:
  // Receives a JSON array of chat.completion.chunk objects.
  using JSONCallback = std::function<void(const std::string& chunks_json)>;
  // Turns the bytes of an encoded image (PNG, JPEG, ...) into prompt embedding rows held by the model
  // backend; returns (embedding handle, number of rows). Counterpart of the image path of the reference's
  // JSON FFI (cpp/json_ffi/image_utils.cc decodes the data URL, the model's image_embed function makes the
  // rows); decoding the pixels and running the vision tower are the host's part here.
  using ImageEmbedder = std::function<std::pair<int64_t, int32_t>(const std::string& image_bytes)>;
  void SetImageEmbedder(ImageEmbedder fn) { image_embedder_ = std::move(fn); }
  // Bytes of a "data:<mime>;base64,<payload>" URL; throws on anything else.
  static std::string DecodeDataURL(const std::string& url);

  JsonFFIEngine(ThreadedEngine::EngineFactory factory, std::shared_ptr<Tokenizer> tokenizer,
                std::string conv_template_json, std::string model_name, JSONCallback callback);

  // Returns false (see GetLastError) when the request is malformed.
  bool ChatCompletion(const std::string& request_json, const std::string& request_id);
  bool Abort(const std::string& request_id);
  std::string GetLastError();
  void Reload(const std::string& engine_config_json) { engine_.Reload(engine_config_json); }
  void Unload() { engine_.Unload(); }
  void Reset() { engine_.Reset(); }
  void RunBackgroundLoop() { engine_.RunBackgroundLoop(); }
  void RunBackgroundStreamBackLoop() { engine_.RunBackgroundStreamBackLoop(); }
  void ExitBackgroundLoop() { engine_.ExitBackgroundLoop(); }
  std::string JSONMetrics() { return engine_.JSONMetrics(); }

 private:
  struct RequestState {
    std::vector<TextStreamer> streamers;  // one per parallel choice
    std::vector<bool> sent_role;
    bool include_usage = false;
  };
  void OnOutputs(std::vector<RequestStreamOutput> outs);

  std::shared_ptr<Tokenizer> tokenizer_;
  std::string conv_json_, model_;
  JSONCallback callback_;
  ImageEmbedder image_embedder_;
  std::mutex mu_;
  std::unordered_map<std::string, RequestState> states_;
  std::string last_error_;
  ThreadedEngine engine_;  // last: its threads call back into the members above
};

}  // namespace mlcb
