#include "tokenizer.h"

#include <algorithm>
#include <stdexcept>

#include "json.h"

namespace mlcb {

// ------------------------------------------------------------------ info
std::string TokenizerInfo::AsJSON() const {
  json::Object o;
  o["token_postproc_method"] = token_postproc_method;
  o["prepend_space_in_encode"] = prepend_space_in_encode;
  o["strip_space_in_decode"] = strip_space_in_decode;
  return json::Value(std::move(o)).dump();
}

TokenizerInfo TokenizerInfo::FromJSON(const std::string& s) {
  TokenizerInfo info;
  json::Value v = json::parse(s);
  const json::Object& o = v.as_object();
  info.token_postproc_method = json::get_or<std::string>(o, "token_postproc_method", "byte_fallback");
  info.prepend_space_in_encode = json::get_or<bool>(o, "prepend_space_in_encode", false);
  info.strip_space_in_decode = json::get_or<bool>(o, "strip_space_in_decode", false);
  return info;
}

static void ForEachComponent(const json::Value* section, const char* list_key,
                             const std::function<void(const json::Object&)>& fn) {
  if (!section || !section->is_object()) return;
  const json::Object& o = section->as_object();
  if (json::get_or<std::string>(o, "type", "") == "Sequence") {
    if (auto* lst = o.find(list_key); lst && lst->is_array())
      for (auto& e : lst->as_array())
        if (e.is_object()) fn(e.as_object());
  } else {
    fn(o);
  }
}

TokenizerInfo TokenizerInfo::Detect(const std::string& tokenizer_json) {
  TokenizerInfo info;
  json::Value root = json::parse(tokenizer_json);
  if (!root.is_object()) return info;
  const json::Object& o = root.as_object();
  ForEachComponent(o.find("decoder"), "decoders", [&](const json::Object& d) {
    std::string type = json::get_or<std::string>(d, "type", "");
    if (type == "ByteLevel") info.token_postproc_method = "byte_level";
    else if (type == "ByteFallback") info.token_postproc_method = "byte_fallback";
    else if (type == "Strip" && json::get_or<std::string>(d, "content", "") == " " &&
             json::get_or<int>(d, "start", 0) == 1 && json::get_or<int>(d, "stop", 0) == 0)
      info.strip_space_in_decode = true;
  });
  ForEachComponent(o.find("normalizer"), "normalizers", [&](const json::Object& n) {
    if (json::get_or<std::string>(n, "type", "") == "Prepend" &&
        json::get_or<std::string>(n, "prepend", "") == "\xE2\x96\x81")
      info.prepend_space_in_encode = true;
  });
  return info;
}

// ------------------------------------------------------------------ token post-processing
static int HexVal(char c) {
  if (c >= '0' && c <= '9') return c - '0';
  if (c >= 'a' && c <= 'f') return c - 'a' + 10;
  if (c >= 'A' && c <= 'F') return c - 'A' + 10;
  return -1;
}

// GPT-2 byte <-> unicode table: printable bytes map to themselves, the rest to U+0100.. in order.
static const std::unordered_map<uint32_t, uint8_t>& ByteLevelInverse() {
  static const std::unordered_map<uint32_t, uint8_t> table = [] {
    std::unordered_map<uint32_t, uint8_t> m;
    int extra = 0;
    for (int b = 0; b < 256; ++b) {
      bool printable = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      if (printable) m[static_cast<uint32_t>(b)] = static_cast<uint8_t>(b);
      else m[256u + static_cast<uint32_t>(extra++)] = static_cast<uint8_t>(b);
    }
    return m;
  }();
  return table;
}

static bool NextCodepoint(const std::string& s, size_t* pos, uint32_t* cp) {
  unsigned char c = static_cast<unsigned char>(s[*pos]);
  int n = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 0;
  if (n == 0 || *pos + n > s.size()) return false;
  uint32_t v = n == 1 ? c : c & (0xFF >> (n + 1));
  for (int i = 1; i < n; ++i) {
    unsigned char cc = static_cast<unsigned char>(s[*pos + i]);
    if ((cc & 0xC0) != 0x80) return false;
    v = (v << 6) | (cc & 0x3F);
  }
  *pos += n;
  *cp = v;
  return true;
}

std::string PostProcessToken(const std::string& token, const std::string& method) {
  if (method == "byte_fallback") {
    if (token.size() == 6 && token.compare(0, 3, "<0x") == 0 && token[5] == '>') {
      int hi = HexVal(token[3]), lo = HexVal(token[4]);
      if (hi >= 0 && lo >= 0) return std::string(1, static_cast<char>(hi * 16 + lo));
    }
    std::string out;
    out.reserve(token.size());
    for (size_t i = 0; i < token.size();) {
      if (token.compare(i, 3, "\xE2\x96\x81") == 0) {
        out.push_back(' ');
        i += 3;
      } else {
        out.push_back(token[i++]);
      }
    }
    return out;
  }
  if (method == "byte_level") {
    const auto& inv = ByteLevelInverse();
    std::string out;
    size_t pos = 0;
    while (pos < token.size()) {
      uint32_t cp;
      size_t save = pos;
      if (!NextCodepoint(token, &pos, &cp)) return token;  // not byte-level text: keep as is
      auto it = inv.find(cp);
      if (it == inv.end()) return token;  // e.g. an added special token with other characters
      (void)save;
      out.push_back(static_cast<char>(it->second));
    }
    return out;
  }
  throw std::runtime_error("Unknown token post-processing method " + method);
}

// ------------------------------------------------------------------ Tokenizer
Tokenizer::Tokenizer(std::vector<std::string> raw_vocab, TokenizerInfo info, EncodeFn encode,
                     std::vector<int32_t> special_token_ids)
    : raw_(std::move(raw_vocab)), info_(std::move(info)), encode_(std::move(encode)) {
  special_.assign(raw_.size(), false);
  for (int32_t id : special_token_ids)
    if (id >= 0 && id < static_cast<int32_t>(raw_.size())) special_[id] = true;
  table_.reserve(raw_.size());
  for (size_t i = 0; i < raw_.size(); ++i) {
    table_.push_back(special_[i] ? raw_[i] : PostProcessToken(raw_[i], info_.token_postproc_method));
    raw_index_.emplace(raw_[i], static_cast<int32_t>(i));
  }
}

std::vector<int32_t> Tokenizer::Encode(const std::string& text) const {
  if (!encode_) throw std::runtime_error("Tokenizer: no encoder attached");
  return encode_(text);
}

std::vector<int32_t> Tokenizer::EncodeNoPrependSpace(const std::string& text) const {
  if (!info_.prepend_space_in_encode) return Encode(text);
  // a sentinel byte takes the prepended space; everything up to and including it is dropped
  std::vector<int32_t> ids = Encode(std::string("\x01") + text);
  for (size_t i = 0; i < ids.size(); ++i) {
    const std::string& bytes = TokenBytes(ids[i]);
    if (!bytes.empty() && bytes.back() == '\x01') {
      ids.erase(ids.begin(), ids.begin() + static_cast<std::ptrdiff_t>(i) + 1);
      return ids;
    }
  }
  return Encode(text);  // the sentinel did not survive as a token of its own
}

const std::vector<bool>& Tokenizer::PrefixTokenMask() const {
  if (!prefix_mask_.empty() || table_.empty()) return prefix_mask_;
  std::vector<bool> mask(table_.size(), false);
  std::vector<int32_t> order(table_.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = static_cast<int32_t>(i);
  std::sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return table_[a] < table_[b]; });
  for (size_t i = 0; i + 1 < order.size(); ++i) {
    const std::string& cur = table_[order[i]];
    const std::string& nxt = table_[order[i + 1]];
    if (cur.size() <= nxt.size() && nxt.compare(0, cur.size(), cur) == 0) mask[order[i]] = true;
  }
  prefix_mask_ = std::move(mask);
  return prefix_mask_;
}

const std::string& Tokenizer::TokenBytes(int32_t id) const {
  if (id < 0 || id >= static_cast<int32_t>(table_.size())) return empty_;
  return table_[id];
}

bool Tokenizer::IsSpecial(int32_t id) const {
  return id >= 0 && id < static_cast<int32_t>(special_.size()) && special_[id];
}

int32_t Tokenizer::TokenToId(const std::string& raw_token) const {
  auto it = raw_index_.find(raw_token);
  return it == raw_index_.end() ? -1 : it->second;
}

const std::string& Tokenizer::IdToRawToken(int32_t id) const {
  if (id < 0 || id >= static_cast<int32_t>(raw_.size())) return empty_;
  return raw_[id];
}

// Replaces invalid UTF-8 by U+FFFD; with `final == false` an incomplete trailing character is left
// in `*rest` instead.
static std::string SanitizeUtf8(const std::string& in, bool final, std::string* rest) {
  std::string out;
  size_t i = 0;
  while (i < in.size()) {
    unsigned char c = static_cast<unsigned char>(in[i]);
    int n = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 0;
    if (n == 0) {
      out += "\xEF\xBF\xBD";
      ++i;
      continue;
    }
    if (i + n > in.size()) {
      // possibly incomplete: check that what we have are continuation bytes
      bool plausible = true;
      for (size_t j = i + 1; j < in.size(); ++j)
        plausible &= (static_cast<unsigned char>(in[j]) & 0xC0) == 0x80;
      if (plausible && !final) {
        if (rest) *rest = in.substr(i);
        return out;
      }
      out += "\xEF\xBF\xBD";
      ++i;
      continue;
    }
    bool ok = true;
    for (int j = 1; j < n; ++j) ok &= (static_cast<unsigned char>(in[i + j]) & 0xC0) == 0x80;
    if (ok) {
      out.append(in, i, n);
      i += n;
    } else {
      out += "\xEF\xBF\xBD";
      ++i;
    }
  }
  if (rest) rest->clear();
  return out;
}

std::string Tokenizer::Decode(const std::vector<int32_t>& ids) const {
  std::string bytes;
  for (int32_t id : ids) bytes += TokenBytes(id);
  if (info_.strip_space_in_decode && !bytes.empty() && bytes[0] == ' ') bytes.erase(0, 1);
  return SanitizeUtf8(bytes, true, nullptr);
}

// ------------------------------------------------------------------ TextStreamer
std::string TextStreamer::Drain(bool final) {
  std::string rest;
  std::string out = SanitizeUtf8(pending_, final, &rest);
  pending_ = rest;
  if (at_start_ && !out.empty()) {
    if (tok_->info().strip_space_in_decode && out[0] == ' ') out.erase(0, 1);
    at_start_ = false;
  }
  return out;
}

std::string TextStreamer::Put(const std::vector<int32_t>& delta_tokens) {
  if (finished_) throw std::runtime_error("TextStreamer: put after finish");
  for (int32_t t : delta_tokens) pending_ += tok_->TokenBytes(t);
  return Drain(false);
}

std::string TextStreamer::Finish() {
  finished_ = true;
  return Drain(true);
}

// ------------------------------------------------------------------ StopStrHandler
StopStrHandler::StopStrHandler(std::vector<std::string> stop_strs, std::shared_ptr<const Tokenizer> tok)
    : stops_(std::move(stop_strs)), tok_(std::move(tok)) {
  stops_.erase(std::remove_if(stops_.begin(), stops_.end(), [](const std::string& s) { return s.empty(); }),
               stops_.end());
  for (auto& s : stops_) max_stop_len_ = std::max(max_stop_len_, s.size());
}

std::vector<int32_t> StopStrHandler::Put(int32_t token_id) {
  std::vector<int32_t> released;
  if (stop_triggered_) return released;
  if (stops_.empty()) {
    released.push_back(token_id);
    return released;
  }
  pending_text_ += tok_->TokenBytes(token_id);
  pending_tokens_.push_back(token_id);
  pending_ends_.push_back(pending_text_.size());
  // 1. a complete stop string inside the pending text?
  size_t match_pos = std::string::npos;
  for (auto& s : stops_) {
    size_t p = pending_text_.find(s);
    if (p != std::string::npos && p < match_pos) match_pos = p;
  }
  size_t keep_from;  // bytes from this offset on must stay pending
  if (match_pos != std::string::npos) {
    stop_triggered_ = true;
    keep_from = match_pos;
  } else {
    // 2. longest suffix of the pending text that is a proper prefix of a stop string
    size_t hold = 0;
    size_t lim = std::min(pending_text_.size(), max_stop_len_ > 0 ? max_stop_len_ - 1 : 0);
    for (size_t len = lim; len > 0; --len) {
      const char* suffix = pending_text_.data() + pending_text_.size() - len;
      bool hit = false;
      for (auto& s : stops_)
        if (s.size() > len && s.compare(0, len, suffix, len) == 0) {
          hit = true;
          break;
        }
      if (hit) {
        hold = len;
        break;
      }
    }
    keep_from = pending_text_.size() - hold;
  }
  // release every token that ends at or before keep_from
  size_t n_release = 0;
  while (n_release < pending_tokens_.size() && pending_ends_[n_release] <= keep_from) ++n_release;
  if (n_release > 0) {
    released.assign(pending_tokens_.begin(), pending_tokens_.begin() + n_release);
    size_t cut = pending_ends_[n_release - 1];
    pending_tokens_.erase(pending_tokens_.begin(), pending_tokens_.begin() + n_release);
    pending_ends_.erase(pending_ends_.begin(), pending_ends_.begin() + n_release);
    for (auto& e : pending_ends_) e -= cut;
    pending_text_.erase(0, cut);
  }
  if (stop_triggered_) {
    pending_tokens_.clear();
    pending_ends_.clear();
    pending_text_.clear();
  }
  return released;
}

std::vector<int32_t> StopStrHandler::Finish() {
  std::vector<int32_t> out;
  out.swap(pending_tokens_);
  pending_ends_.clear();
  pending_text_.clear();
  return out;
}

}  // namespace mlcb
