// ThreadedEngine: an Engine driven by a background loop fed through an instruction queue, with a
// second loop that batches stream outputs back to the frontend so the engine thread never runs
// frontend code. Reload / unload / reset are synchronous for the caller.
#include <algorithm>

#include "engine.h"

namespace mlcb {

ThreadedEngine::ThreadedEngine(EngineFactory factory, StreamCallback frontend_callback)
    : factory_(std::move(factory)), frontend_callback_(std::move(frontend_callback)) {}

ThreadedEngine::~ThreadedEngine() { ExitBackgroundLoop(); }

void ThreadedEngine::Reload(const std::string& engine_config_json) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    queue_.push_back({Kind::kReload, nullptr, engine_config_json});
    std::lock_guard<std::mutex> l2(reload_mu_);
    reload_done_ = false;
    error_.clear();
  }
  cv_.notify_one();
  std::unique_lock<std::mutex> lock(reload_mu_);
  reload_cv_.wait(lock, [this] { return reload_done_ || exit_.load(); });
  if (!error_.empty()) throw std::runtime_error(error_);
}

void ThreadedEngine::Unload() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    queue_.push_back({Kind::kUnload, nullptr, ""});
    std::lock_guard<std::mutex> l2(reload_mu_);
    unload_done_ = false;
  }
  cv_.notify_one();
  std::unique_lock<std::mutex> lock(reload_mu_);
  reload_cv_.wait(lock, [this] { return unload_done_ || exit_.load(); });
}

void ThreadedEngine::Reset() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    queue_.push_back({Kind::kReset, nullptr, ""});
    std::lock_guard<std::mutex> l2(reload_mu_);
    reset_done_ = false;
  }
  cv_.notify_one();
  std::unique_lock<std::mutex> lock(reload_mu_);
  reload_cv_.wait(lock, [this] { return reset_done_ || exit_.load(); });
}

void ThreadedEngine::AddRequest(Request request) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    queue_.push_back({Kind::kAddRequest, std::make_shared<Request>(std::move(request)), ""});
  }
  cv_.notify_one();
}

void ThreadedEngine::AbortRequest(const std::string& request_id) {
  {
    std::lock_guard<std::mutex> lock(mu_);
    queue_.push_back({Kind::kAbortRequest, nullptr, request_id});
  }
  cv_.notify_one();
  // an aborted request produces no final output: drop what the stream-back thread gathered for it
  std::lock_guard<std::mutex> lock(acc_mu_);
  acc_.erase(request_id);
}

void ThreadedEngine::HandleReload(const std::string& cfg) {
  std::string err;
  try {
    auto cb = [this](std::vector<RequestStreamOutput> outs) {
      {
        std::lock_guard<std::mutex> lock(sb_mu_);
        for (auto& o : outs) sb_queue_.push_back(std::move(o));
        pending_outputs_.fetch_add(1);
      }
      sb_cv_.notify_one();
    };
    std::unique_ptr<Engine> fresh = factory_(cfg, cb);
    std::lock_guard<std::mutex> lock(engine_mu_);
    engine_ = std::move(fresh);
  } catch (const std::exception& e) {
    err = e.what();
  }
  {
    std::lock_guard<std::mutex> lock(reload_mu_);
    error_ = err;
    reload_done_ = true;
  }
  reload_cv_.notify_all();
}

void ThreadedEngine::HandleUnload() {
  {
    std::lock_guard<std::mutex> lock(engine_mu_);
    if (engine_) engine_->AbortAllRequests();
    engine_.reset();
  }
  {
    std::lock_guard<std::mutex> lock(reload_mu_);
    unload_done_ = true;
  }
  reload_cv_.notify_all();
}

void ThreadedEngine::RunBackgroundLoop() {
  while (!exit_.load()) {
    std::vector<Instruction> local;
    {
      std::unique_lock<std::mutex> lock(mu_);
      engine_waiting_.store(true);
      cv_.wait(lock, [this] {
        return exit_.load() || !queue_.empty() || (engine_ && !engine_->Empty());
      });
      engine_waiting_.store(false);
      local.swap(queue_);
    }
    if (exit_.load()) break;
    for (auto& ins : local) {
      try {
        switch (ins.kind) {
          case Kind::kAddRequest:
            if (engine_) engine_->AddRequest(std::move(*ins.request));
            break;
          case Kind::kAbortRequest:
            if (engine_) engine_->AbortRequest(ins.arg);
            break;
          case Kind::kReload:
            HandleReload(ins.arg);
            break;
          case Kind::kUnload:
            HandleUnload();
            break;
          case Kind::kReset: {
            if (engine_) engine_->Reset();
            {
              std::lock_guard<std::mutex> lock(reload_mu_);
              reset_done_ = true;
            }
            reload_cv_.notify_all();
            break;
          }
          case Kind::kDebugCall:
            break;
        }
      } catch (const std::exception& e) {
        // a bad request must not take the engine thread down: report it as a failed stream output
        if (ins.kind == Kind::kAddRequest && ins.request) {
          RequestStreamOutput out;
          out.request_id = ins.request->id;
          const int n = std::max(1, ins.request->cfg.n);
          out.group_delta_token_ids.resize(n);
          out.group_delta_logprob_json_strs.resize(n);
          out.group_finish_reason.assign(n, "error");
          out.group_extra_prefix_string.assign(n, e.what());
          out.request_final_usage_json_str = "{\"prompt_tokens\":0,\"completion_tokens\":0,\"total_tokens\":0}";
          {
            std::lock_guard<std::mutex> lock(sb_mu_);
            sb_queue_.push_back(std::move(out));
          }
          sb_cv_.notify_one();
        }
        std::lock_guard<std::mutex> lock(reload_mu_);
        error_ = e.what();
      }
    }
    if (engine_ && !engine_->Empty()) {
      try {
        engine_->Step();
      } catch (const std::exception& e) {
        {
          std::lock_guard<std::mutex> lock(reload_mu_);
          error_ = std::string("engine step failed: ") + e.what();
        }
        // fail every in-flight request rather than spinning on a broken step
        engine_->AbortAllRequests();
        {
          std::lock_guard<std::mutex> lock(acc_mu_);
          acc_.clear();  // their gathered outputs will never be completed
        }
        RequestStreamOutput out;
        out.request_id = "";
        out.group_finish_reason = {"error"};
        out.group_extra_prefix_string = {e.what()};
        out.group_delta_token_ids.resize(1);
        out.group_delta_logprob_json_strs.resize(1);
        {
          std::lock_guard<std::mutex> lock(sb_mu_);
          sb_queue_.push_back(std::move(out));
        }
        sb_cv_.notify_one();
      }
    }
  }
}

void ThreadedEngine::RunBackgroundStreamBackLoop() {
  while (!exit_.load()) {
    std::vector<RequestStreamOutput> local;
    {
      std::unique_lock<std::mutex> lock(sb_mu_);
      sb_waiting_.store(true);
      sb_cv_.wait(lock, [this] { return exit_.load() || !sb_queue_.empty(); });
      sb_waiting_.store(false);
      local.swap(sb_queue_);
    }
    if (exit_.load()) break;
    std::vector<RequestStreamOutput> forward;
    forward.reserve(local.size());
    for (auto& out : local)
      if (Accumulate(&out)) forward.push_back(std::move(out));
    if (!forward.empty() && frontend_callback_) frontend_callback_(std::move(forward));
  }
}

void ThreadedEngine::AccumulateOutputs(const std::string& request_id, int num_choices,
                                       std::shared_ptr<const Tokenizer> tokenizer) {
  OutputAccumulator acc;
  const int n = std::max(1, num_choices);
  acc.merged.request_id = request_id;
  acc.merged.group_delta_token_ids.resize(n);
  acc.merged.group_delta_logprob_json_strs.resize(n);
  acc.merged.group_finish_reason.assign(n, "");
  acc.merged.group_extra_prefix_string.assign(n, "");
  acc.merged.text_is_final = true;
  for (int i = 0; i < n; ++i) acc.streamers.emplace_back(tokenizer);
  acc.finished.assign(n, false);
  std::lock_guard<std::mutex> lock(acc_mu_);
  acc_[request_id] = std::move(acc);
}

bool ThreadedEngine::Accumulate(RequestStreamOutput* out) {
  std::lock_guard<std::mutex> lock(acc_mu_);
  auto it = acc_.find(out->request_id);
  if (it == acc_.end()) return true;
  OutputAccumulator& acc = it->second;
  const size_t n = acc.streamers.size();
  bool error = false;
  for (size_t i = 0; i < n && i < out->group_delta_token_ids.size(); ++i) {
    if (acc.finished[i]) continue;
    const std::string& reason = i < out->group_finish_reason.size() ? out->group_finish_reason[i] : std::string();
    if (reason == "error") {
      error = true;
      break;
    }
    std::string& text = acc.merged.group_extra_prefix_string[i];
    if (i < out->group_extra_prefix_string.size()) text += out->group_extra_prefix_string[i];
    const std::vector<int32_t>& ids = out->group_delta_token_ids[i];
    if (!ids.empty()) {
      text += acc.streamers[i].Put(ids);
      acc.merged.group_delta_token_ids[i].insert(acc.merged.group_delta_token_ids[i].end(), ids.begin(), ids.end());
    }
    if (i < out->group_delta_logprob_json_strs.size())
      for (auto& s : out->group_delta_logprob_json_strs[i]) acc.merged.group_delta_logprob_json_strs[i].push_back(s);
    if (!reason.empty()) {
      text += acc.streamers[i].Finish();
      acc.merged.group_finish_reason[i] = reason;
      acc.finished[i] = true;
    }
  }
  if (error) {  // pass the error through as it is
    acc_.erase(it);
    return true;
  }
  if (out->request_final_usage_json_str.empty()) return false;
  acc.merged.request_final_usage_json_str = out->request_final_usage_json_str;
  *out = std::move(acc.merged);
  acc_.erase(it);
  return true;
}

void ThreadedEngine::ExitBackgroundLoop() {
  exit_.store(true);
  {
    std::lock_guard<std::mutex> lock(mu_);
  }
  cv_.notify_all();
  {
    std::lock_guard<std::mutex> lock(sb_mu_);
  }
  sb_cv_.notify_all();
  reload_cv_.notify_all();
}

std::string ThreadedEngine::JSONMetrics() {
  std::lock_guard<std::mutex> lock(engine_mu_);
  return engine_ ? engine_->JSONMetrics() : "{}";
}

std::string ThreadedEngine::CompleteEngineConfigJSON() {
  std::lock_guard<std::mutex> lock(engine_mu_);
  return engine_ ? engine_->Config().AsJSON().dump() : "{}";
}

GenerationConfig ThreadedEngine::DefaultGenerationConfig() {
  std::lock_guard<std::mutex> lock(engine_mu_);
  return engine_ ? engine_->DefaultGenerationConfig() : GenerationConfig();
}

std::string ThreadedEngine::last_error() {
  std::lock_guard<std::mutex> lock(reload_mu_);
  return error_;
}

}  // namespace mlcb
