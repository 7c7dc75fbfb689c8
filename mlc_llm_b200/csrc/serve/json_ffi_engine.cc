#include "json_ffi_engine.h"

#include <chrono>

#include "conv_template.h"
#include "json.h"

namespace mlcb {

namespace {
int64_t UnixSeconds() {
  return std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch())
      .count();
}
}  // namespace

std::string JsonFFIEngine::DecodeDataURL(const std::string& url) {
  const std::string marker = ";base64,";
  const size_t at = url.find(marker);
  if (url.compare(0, 5, "data:") != 0 || at == std::string::npos)
    throw std::runtime_error("image_url must be a data URL (data:image/...;base64,...)");
  std::string out;
  out.reserve((url.size() - at) * 3 / 4);
  uint32_t acc = 0;
  int bits = 0;
  for (size_t i = at + marker.size(); i < url.size(); ++i) {
    const unsigned char ch = static_cast<unsigned char>(url[i]);
    int v;
    if (ch >= 'A' && ch <= 'Z') v = ch - 'A';
    else if (ch >= 'a' && ch <= 'z') v = ch - 'a' + 26;
    else if (ch >= '0' && ch <= '9') v = ch - '0' + 52;
    else if (ch == '+' || ch == '-') v = 62;
    else if (ch == '/' || ch == '_') v = 63;
    else if (ch == '=' || ch == '\n' || ch == '\r' || ch == ' ') continue;
    else throw std::runtime_error("image_url: character outside the base64 alphabet");
    acc = (acc << 6) | static_cast<uint32_t>(v);
    bits += 6;
    if (bits >= 8) {
      bits -= 8;
      out.push_back(static_cast<char>((acc >> bits) & 0xff));
    }
  }
  if (out.empty()) throw std::runtime_error("image_url: empty payload");
  return out;
}

JsonFFIEngine::JsonFFIEngine(ThreadedEngine::EngineFactory factory, std::shared_ptr<Tokenizer> tokenizer,
                             std::string conv_template_json, std::string model_name, JSONCallback callback)
    : tokenizer_(std::move(tokenizer)),
      conv_json_(std::move(conv_template_json)),
      model_(std::move(model_name)),
      callback_(std::move(callback)),
      engine_(std::move(factory), [this](std::vector<RequestStreamOutput> outs) { OnOutputs(std::move(outs)); }) {}

std::string JsonFFIEngine::GetLastError() {
  std::lock_guard<std::mutex> lock(mu_);
  return last_error_;
}

bool JsonFFIEngine::ChatCompletion(const std::string& request_json, const std::string& request_id) {
  try {
    json::Value root = json::parse(request_json);
    if (!root.is_object()) throw std::runtime_error("the request must be a JSON object");
    json::Object& req = root.as_object();
    const json::Value* messages = req.find("messages");
    if (messages == nullptr || !messages->is_array() || messages->as_array().empty())
      throw std::runtime_error("\"messages\" must be a non-empty array");
    // 1. conversation template -> prompt text -> token ids
    std::vector<std::string> image_urls;
    const std::string prompt = RenderConversation(conv_json_, messages->dump(), &image_urls);
    if (!image_urls.empty() && !image_embedder_)
      throw std::runtime_error("this model does not take image inputs");
    Request request;
    request.id = request_id;
    json::Value conv = json::parse(conv_json_);
    std::vector<int32_t> prefix_ids;
    if (conv.is_object()) {
      if (const json::Value* pre = conv.as_object().find("system_prefix_token_ids"); pre && pre->is_array())
        for (auto& v : pre->as_array()) prefix_ids.push_back(static_cast<int32_t>(v.as_int()));
    }
    // text pieces between the image placeholders become token items, the images embedding items
    const std::string mark = kImagePlaceholder;
    size_t from = 0, image = 0;
    while (true) {
      const size_t at = image < image_urls.size() ? prompt.find(mark, from) : std::string::npos;
      const std::string piece = prompt.substr(from, at == std::string::npos ? std::string::npos : at - from);
      InputItem item;
      if (!piece.empty()) item.tokens = tokenizer_->Encode(piece);
      if (from == 0) item.tokens.insert(item.tokens.begin(), prefix_ids.begin(), prefix_ids.end());
      if (!item.tokens.empty()) {
        request.prompt_tokens += static_cast<int64_t>(item.tokens.size());
        request.inputs.push_back(std::move(item));
      }
      if (at == std::string::npos) break;
      const auto rows = image_embedder_(DecodeDataURL(image_urls[image++]));
      if (rows.first < 0 || rows.second <= 0) throw std::runtime_error("the image could not be embedded");
      InputItem img;
      img.kind = 1;
      img.embed_handle = rows.first;
      img.embed_len = rows.second;
      request.prompt_tokens += rows.second;
      request.inputs.push_back(std::move(img));
      from = at + mark.size();
    }
    if (request.inputs.empty()) throw std::runtime_error("the rendered prompt is empty");
    // 2. generation config: request fields over the model defaults, plus the template's stop rules
    json::Object gen;
    for (auto& m : req.members()) {
      if (m.first == "messages" || m.first == "model" || m.first == "stream" || m.first == "stream_options" ||
          m.first == "tools" || m.first == "tool_choice" || m.first == "user" || m.first == "stop")
        continue;
      if (!m.second.is_null()) gen[m.first] = m.second;
    }
    json::Array stop_strs, stop_ids;
    if (const json::Value* stop = req.find("stop")) {
      if (stop->is_string()) stop_strs.push_back(*stop);
      if (stop->is_array())
        for (auto& s : stop->as_array()) stop_strs.push_back(s);
    }
    if (conv.is_object()) {
      if (const json::Value* s = conv.as_object().find("stop_str"); s && s->is_array())
        for (auto& v : s->as_array()) stop_strs.push_back(v);
      if (const json::Value* s = conv.as_object().find("stop_token_ids"); s && s->is_array())
        for (auto& v : s->as_array()) stop_ids.push_back(v);
    }
    gen["stop_strs"] = json::Value(stop_strs);
    gen["stop_token_ids"] = json::Value(stop_ids);
    request.cfg = GenerationConfig::FromJSON(json::Value(gen).dump(), engine_.DefaultGenerationConfig());
    RequestState st;
    for (int i = 0; i < request.cfg.n; ++i) {
      st.streamers.emplace_back(tokenizer_);
      st.sent_role.push_back(false);
    }
    if (const json::Value* so = req.find("stream_options"); so && so->is_object()) {
      if (const json::Value* iu = so->as_object().find("include_usage"); iu && iu->is_bool())
        st.include_usage = iu->as_bool();
    }
    {
      std::lock_guard<std::mutex> lock(mu_);
      if (states_.count(request_id)) throw std::runtime_error("the request id " + request_id + " already exists");
      states_.emplace(request_id, std::move(st));
    }
    engine_.AddRequest(std::move(request));
    return true;
  } catch (const std::exception& e) {
    std::lock_guard<std::mutex> lock(mu_);
    last_error_ = e.what();
    return false;
  }
}

bool JsonFFIEngine::Abort(const std::string& request_id) {
  engine_.AbortRequest(request_id);
  std::lock_guard<std::mutex> lock(mu_);
  states_.erase(request_id);
  return true;
}

void JsonFFIEngine::OnOutputs(std::vector<RequestStreamOutput> outs) {
  json::Array chunks;
  for (auto& out : outs) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = states_.find(out.request_id);
    if (it == states_.end()) continue;
    RequestState& st = it->second;
    const bool final_usage = !out.request_final_usage_json_str.empty();
    json::Array choices;
    for (size_t i = 0; i < out.group_delta_token_ids.size() && i < st.streamers.size(); ++i) {
      std::string text = out.group_extra_prefix_string.size() > i ? out.group_extra_prefix_string[i] : "";
      text += st.streamers[i].Put(out.group_delta_token_ids[i]);
      const std::string& reason = out.group_finish_reason[i];
      if (!reason.empty()) text += st.streamers[i].Finish();
      if (text.empty() && reason.empty()) continue;
      json::Object delta;
      delta["content"] = json::Value(text);
      delta["role"] = json::Value(std::string("assistant"));
      json::Object choice;
      choice["index"] = json::Value(static_cast<int64_t>(i));
      choice["delta"] = json::Value(delta);
      choice["finish_reason"] = reason.empty() ? json::Value() : json::Value(reason);
      if (out.group_delta_logprob_json_strs.size() > i && !out.group_delta_logprob_json_strs[i].empty()) {
        json::Array content;
        for (auto& s : out.group_delta_logprob_json_strs[i]) content.push_back(json::parse(s));
        json::Object lp;
        lp["content"] = json::Value(content);
        choice["logprobs"] = json::Value(lp);
      }
      choices.push_back(json::Value(choice));
    }
    auto make_chunk = [&](json::Array ch, const json::Value& usage) {
      json::Object chunk;
      chunk["id"] = json::Value(out.request_id);
      chunk["object"] = json::Value(std::string("chat.completion.chunk"));
      chunk["created"] = json::Value(UnixSeconds());
      chunk["model"] = json::Value(model_);
      chunk["system_fingerprint"] = json::Value(std::string(""));
      chunk["choices"] = json::Value(std::move(ch));
      chunk["usage"] = usage;
      return json::Value(chunk);
    };
    if (!choices.empty()) chunks.push_back(make_chunk(std::move(choices), json::Value()));
    if (final_usage) {
      if (st.include_usage) chunks.push_back(make_chunk(json::Array(), json::parse(out.request_final_usage_json_str)));
      states_.erase(it);
    }
  }
  if (!chunks.empty() && callback_) callback_(json::Value(chunks).dump());
}

}  // namespace mlcb
