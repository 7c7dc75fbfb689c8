// Conversation-template rendering in C++, used by the JSON FFI entry point so that
// embedders without Python get the same prompts as the Python API.
//
// Behavioural counterpart: cpp/json_ffi/conv_template.cc:224-416 and
// python/mlc_llm/protocol/conversation_protocol.py:115-208.
#pragma once
#include <string>
#include <vector>

namespace mlcb {

// Stands in the rendered prompt for each image content part (in order of appearance).
extern const char* const kImagePlaceholder;

// conv_json: a conversation template object (fields of mlc-chat-config.json "conv_template").
// messages_json: OpenAI-style [{"role":..., "content": str | [{"type":"text","text":...}] | null}].
// A trailing generation prompt (assistant role with empty content) is appended unless the last
// message already is an assistant message with null content.
// image_urls: when non-null, {"type":"image_url","image_url":{"url":...}} (or "image_url": "<url>") parts
// are accepted: the URL is appended to the vector and kImagePlaceholder to the text. When null such a
// part is an error.
std::string RenderConversation(const std::string& conv_json, const std::string& messages_json,
                               std::vector<std::string>* image_urls = nullptr);

}  // namespace mlcb
