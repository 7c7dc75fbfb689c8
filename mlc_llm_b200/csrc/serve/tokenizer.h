// Tokenizer glue: tokenizer-info detection from a HuggingFace tokenizer.json, the post-processed
// token table (raw bytes per token id), table-driven decoding, incremental UTF-8-safe
// detokenisation (TextStreamer) and the stop-string matcher over a token stream (StopStrHandler).
// Encoding is delegated to a callback (the HuggingFace / SentencePiece encoder bound from Python).
//
// Behavioural counterparts: cpp/tokenizers/tokenizers.cc:197-459 (info detection, byte_fallback and
// byte_level post-processing) and cpp/tokenizers/streamer.cc:33-266.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace mlcb {

struct TokenizerInfo {
  std::string token_postproc_method = "byte_fallback";  // or "byte_level"
  bool prepend_space_in_encode = false;
  bool strip_space_in_decode = false;
  std::string AsJSON() const;
  static TokenizerInfo FromJSON(const std::string& s);
  // Inspects the "decoder" and "normalizer" sections of a tokenizer.json document.
  static TokenizerInfo Detect(const std::string& tokenizer_json);
};

// Converts one raw vocabulary entry into the bytes it stands for.
std::string PostProcessToken(const std::string& token, const std::string& method);

class Tokenizer {
 public:
  using EncodeFn = std::function<std::vector<int32_t>(const std::string&)>;
  Tokenizer(std::vector<std::string> raw_vocab, TokenizerInfo info, EncodeFn encode,
            std::vector<int32_t> special_token_ids = {});

  std::vector<int32_t> Encode(const std::string& text) const;
  // Encodes a continuation of earlier text: tokenizers that put a space in front of every input
  // (SentencePiece-style) are kept from doing so here (reference: cpp/tokenizers/tokenizers.cc:78-90).
  std::vector<int32_t> EncodeNoPrependSpace(const std::string& text) const;
  // [id] = the token's bytes are a prefix of another token's bytes (such a token is likely to be
  // re-merged by the next decode step; reference: cpp/tokenizers/tokenizers.cc:104-131).
  const std::vector<bool>& PrefixTokenMask() const;
  std::string Decode(const std::vector<int32_t>& ids) const;  // whole-text decode
  const std::string& TokenBytes(int32_t id) const;
  int64_t VocabSize() const { return static_cast<int64_t>(table_.size()); }
  const std::vector<std::string>& PostprocTokenTable() const { return table_; }
  const TokenizerInfo& info() const { return info_; }
  bool IsSpecial(int32_t id) const;
  int32_t TokenToId(const std::string& raw_token) const;
  const std::string& IdToRawToken(int32_t id) const;

 private:
  std::vector<std::string> raw_;
  std::vector<std::string> table_;
  TokenizerInfo info_;
  EncodeFn encode_;
  std::vector<bool> special_;
  std::unordered_map<std::string, int32_t> raw_index_;
  std::string empty_;
  mutable std::vector<bool> prefix_mask_;
};

class TextStreamer {
 public:
  explicit TextStreamer(std::shared_ptr<const Tokenizer> tok) : tok_(std::move(tok)) {}
  // Returns the text that became certain after these tokens (never splits a UTF-8 character).
  std::string Put(const std::vector<int32_t>& delta_tokens);
  // Flushes whatever is still held back (incomplete bytes become U+FFFD).
  std::string Finish();

 private:
  std::string Drain(bool final);
  std::shared_ptr<const Tokenizer> tok_;
  std::string pending_;
  bool at_start_ = true;
  bool finished_ = false;
};

class StopStrHandler {
 public:
  StopStrHandler(std::vector<std::string> stop_strs, std::shared_ptr<const Tokenizer> tok);
  // Feeds one token; returns the tokens that can be released now.
  std::vector<int32_t> Put(int32_t token_id);
  // Releases the tokens still held back (call when generation ends without a stop string).
  std::vector<int32_t> Finish();
  bool stop_triggered() const { return stop_triggered_; }

 private:
  std::vector<std::string> stops_;
  std::shared_ptr<const Tokenizer> tok_;
  size_t max_stop_len_ = 0;
  std::vector<int32_t> pending_tokens_;
  std::vector<size_t> pending_ends_;  // end offset of each pending token inside pending_text_
  std::string pending_text_;
  bool stop_triggered_ = false;
};

}  // namespace mlcb
