// Engine / request / speculative-decoding metrics and the per-request event trace recorder.
//
// Behavioural counterparts: cpp/serve/metrics.h:28-259 + metrics.cc:25-162 (counter names, usage
// JSON with "extra", prometheus-style labelled entries) and cpp/serve/event_trace_recorder.cc:41-159
// (Chrome trace "B"/"E"/"i" events, tid = request id).
#pragma once
#include <chrono>
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "json.h"

namespace mlcb {

inline double NowSeconds() {
  using namespace std::chrono;
  return duration_cast<duration<double>>(steady_clock::now().time_since_epoch()).count();
}

struct TimeCost {
  double sum = 0;
  int64_t count = 0;
  void Update(double v) {
    sum += v;
    ++count;
  }
  void Reset() { sum = 0; count = 0; }
  json::Value AsJSON() const {
    json::Object o;
    o["count"] = count;
    if (count) o["mean"] = sum / static_cast<double>(count);
    return json::Value(std::move(o));
  }
};

struct SpecDecodeMetrics {
  std::vector<int64_t> draft_count, accept_count;  // per draft position
  void Update(int draft_length, int accepted) {
    if (static_cast<int>(draft_count.size()) < draft_length) {
      draft_count.resize(draft_length, 0);
      accept_count.resize(draft_length, 0);
    }
    for (int i = 0; i < draft_length; ++i) ++draft_count[i];
    for (int i = 0; i < accepted && i < draft_length; ++i) ++accept_count[i];
  }
  void Reset() { draft_count.clear(); accept_count.clear(); }
  bool IsEmpty() const { return draft_count.empty(); }
  json::Value AsJSON() const;
};

struct RequestMetrics {
  int64_t prompt_tokens = 0, completion_tokens = 0, prefill_tokens = 0, decode_tokens = 0,
          jump_forward_tokens = 0;
  double add_time = 0, prefill_end_time = 0, finish_time = 0;
  bool IsComplete() const { return prompt_tokens != 0 && completion_tokens != 0; }
  // OpenAI "usage" object; `include_extra` adds the speed / latency block.
  json::Value AsUsageJSON(bool include_extra = true) const;
};

struct EngineMetrics {
  double engine_prefill_time_sum = 0, engine_decode_time_sum = 0, engine_jump_forward_time_sum = 0;
  int64_t prompt_tokens_sum = 0, completion_tokens_sum = 0, prefill_tokens_sum = 0,
          decode_tokens_sum = 0, jump_forward_tokens_sum = 0;
  RequestMetrics last_finished_request;
  SpecDecodeMetrics spec_decode;
  static constexpr int kMaxBatch = 64;
  std::vector<TimeCost> decode_time_by_batch_size, draft_time_by_batch_size, verify_time_by_batch_size;
  EngineMetrics() { Reset(); }
  void RequestFinishUpdate(const RequestMetrics& m);
  void UpdateDecodeTimeByBatchSize(int bs, double t) { if (bs > 0 && bs <= kMaxBatch) decode_time_by_batch_size[bs].Update(t); }
  void UpdateDraftTimeByBatchSize(int bs, double t) { if (bs > 0 && bs <= kMaxBatch) draft_time_by_batch_size[bs].Update(t); }
  void UpdateVerifyTimeByBatchSize(int bs, double t) { if (bs > 0 && bs <= kMaxBatch) verify_time_by_batch_size[bs].Update(t); }
  json::Value AsJSON() const;
  void Reset();
};

class EventTraceRecorder {
 public:
  void AddEvent(const std::string& request_id, const std::string& event);
  void AddEvent(const std::vector<std::string>& request_ids, const std::string& event);
  // Chrome trace-event JSON (array of events, microsecond timestamps relative to the first event).
  std::string DumpJSON() const;
  void Clear();

 private:
  mutable std::mutex mu_;
  std::vector<std::pair<std::string, std::pair<std::string, double>>> events_;
};

}  // namespace mlcb
