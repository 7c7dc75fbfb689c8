#include "metrics.h"

#include <algorithm>
#include <set>
#include <sstream>

namespace mlcb {

using json::Object;
using json::Value;

static Value IntArray(const std::vector<int64_t>& v) {
  json::Array a;
  for (int64_t x : v) a.emplace_back(x);
  return Value(std::move(a));
}

Value SpecDecodeMetrics::AsJSON() const {
  Object m;
  m["draft_count"] = IntArray(draft_count);
  m["accept_count"] = IntArray(accept_count);
  Object prob, rate, len;
  double running = 0;
  for (size_t i = 0; i < draft_count.size(); ++i) {
    const double p = draft_count[i] ? static_cast<double>(accept_count[i]) / draft_count[i] : 0.0;
    running += p;
    prob["accept_prob{step=" + std::to_string(i) + "}"] = p;
    len["accept_len{step=" + std::to_string(i) + "}"] = running;
    if (i != 0)
      rate["accept_rate{step=" + std::to_string(i) + "}"] =
          accept_count[i - 1] ? static_cast<double>(accept_count[i]) / accept_count[i - 1] : 0.0;
  }
  m["accept_prob"] = Value(std::move(prob));
  m["accept_rate"] = Value(std::move(rate));
  m["accept_len"] = Value(std::move(len));
  return Value(std::move(m));
}

static Object RequestExtra(const RequestMetrics& r) {
  Object m;
  m["prompt_tokens"] = r.prompt_tokens;
  m["completion_tokens"] = r.completion_tokens;
  m["prefill_tokens"] = r.prefill_tokens;
  m["decode_tokens"] = r.decode_tokens;
  m["jump_forward_tokens"] = r.jump_forward_tokens;
  const double prefill_t = r.prefill_end_time - r.add_time;
  const double decode_t = r.finish_time - r.prefill_end_time;
  const double total_t = r.finish_time - r.add_time;
  if (r.prefill_tokens != 0 && prefill_t > 0) m["prefill_tokens_per_s"] = r.prefill_tokens / prefill_t;
  if (r.decode_tokens != 0 && decode_t > 0) m["decode_tokens_per_s"] = r.decode_tokens / decode_t;
  m["end_to_end_latency_s"] = total_t;
  m["ttft_s"] = prefill_t;
  m["inter_token_latency_s"] = r.completion_tokens ? total_t / r.completion_tokens : 0.0;
  return m;
}

Value RequestMetrics::AsUsageJSON(bool include_extra) const {
  Object u;
  u["prompt_tokens"] = prompt_tokens;
  u["completion_tokens"] = completion_tokens;
  u["total_tokens"] = prompt_tokens + completion_tokens;
  if (include_extra) u["extra"] = Value(RequestExtra(*this));
  return Value(std::move(u));
}

void EngineMetrics::Reset() {
  engine_prefill_time_sum = engine_decode_time_sum = engine_jump_forward_time_sum = 0;
  prompt_tokens_sum = completion_tokens_sum = prefill_tokens_sum = decode_tokens_sum =
      jump_forward_tokens_sum = 0;
  last_finished_request = RequestMetrics();
  spec_decode.Reset();
  decode_time_by_batch_size.assign(kMaxBatch + 1, TimeCost());
  draft_time_by_batch_size.assign(kMaxBatch + 1, TimeCost());
  verify_time_by_batch_size.assign(kMaxBatch + 1, TimeCost());
}

void EngineMetrics::RequestFinishUpdate(const RequestMetrics& m) {
  prompt_tokens_sum += m.prompt_tokens;
  prefill_tokens_sum += m.prefill_tokens;
  completion_tokens_sum += m.completion_tokens;
  decode_tokens_sum += m.decode_tokens;
  jump_forward_tokens_sum += m.jump_forward_tokens;
  last_finished_request = m;
}

static Value TimeList(const std::vector<TimeCost>& lst) {
  Object o;
  for (size_t i = 1; i < lst.size(); ++i) {
    if (lst[i].count == 0) continue;
    o["mean{batch_size=" + std::to_string(i) + "}"] = lst[i].sum / lst[i].count;
    o["count{batch_size=" + std::to_string(i) + "}"] = lst[i].count;
  }
  return Value(std::move(o));
}

Value EngineMetrics::AsJSON() const {
  Object m;
  m["engine_prefill_time_sum"] = engine_prefill_time_sum;
  m["engine_decode_time_sum"] = engine_decode_time_sum;
  m["engine_jump_forward_time_sum"] = engine_jump_forward_time_sum;
  m["prompt_tokens_sum"] = prompt_tokens_sum;
  m["completion_tokens_sum"] = completion_tokens_sum;
  m["prefill_tokens_sum"] = prefill_tokens_sum;
  m["decode_tokens_sum"] = decode_tokens_sum;
  m["jump_forward_tokens_sum"] = jump_forward_tokens_sum;
  if (prefill_tokens_sum != 0 && engine_prefill_time_sum > 0)
    m["prefill_tokens_per_s"] = prefill_tokens_sum / engine_prefill_time_sum;
  if (engine_decode_time_sum != 0) m["decode_tokens_per_s"] = decode_tokens_sum / engine_decode_time_sum;
  m["last_finished_request"] = Value(RequestExtra(last_finished_request));
  if (!spec_decode.IsEmpty()) m["spec_decode"] = spec_decode.AsJSON();
  m["decode_time_by_batch_size"] = TimeList(decode_time_by_batch_size);
  m["draft_time_by_batch_size"] = TimeList(draft_time_by_batch_size);
  m["verify_time_by_batch_size"] = TimeList(verify_time_by_batch_size);
  return Value(std::move(m));
}

// ------------------------------------------------------------------ event trace
void EventTraceRecorder::AddEvent(const std::string& request_id, const std::string& event) {
  const double t = NowSeconds();
  std::lock_guard<std::mutex> lock(mu_);
  events_.push_back({request_id, {event, t}});
}

void EventTraceRecorder::AddEvent(const std::vector<std::string>& request_ids, const std::string& event) {
  const double t = NowSeconds();
  std::lock_guard<std::mutex> lock(mu_);
  for (auto& id : request_ids) events_.push_back({id, {event, t}});
}

void EventTraceRecorder::Clear() {
  std::lock_guard<std::mutex> lock(mu_);
  events_.clear();
}

std::string EventTraceRecorder::DumpJSON() const {
  std::lock_guard<std::mutex> lock(mu_);
  json::Array out;
  if (events_.empty()) return "[]";
  double t0 = events_.front().second.second;
  for (auto& e : events_) t0 = std::min(t0, e.second.second);
  for (auto& e : events_) {
    const std::string& name = e.second.first;
    std::string ph = "i", label = name;
    if (name.compare(0, 6, "start ") == 0) {
      ph = "B";
      label = name.substr(6);
    } else if (name.compare(0, 7, "finish ") == 0) {
      ph = "E";
      label = name.substr(7);
    }
    Object ev;
    ev["name"] = label;
    ev["ph"] = ph;
    ev["ts"] = (e.second.second - t0) * 1e6;
    ev["pid"] = 1;
    ev["tid"] = e.first;
    if (ph == "i") ev["s"] = "t";
    out.emplace_back(std::move(ev));
  }
  return Value(std::move(out)).dump();
}

}  // namespace mlcb
