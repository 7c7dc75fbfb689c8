// Conversation-template rendering in C++ (text-only), used by the JSON FFI entry point so that
// embedders without Python get the same prompts as the Python API.
//
// Behavioural counterpart: cpp/json_ffi/conv_template.cc:224-416 and
// python/mlc_llm/protocol/conversation_protocol.py:115-208.
#pragma once
#include <string>

namespace mlcb {

// conv_json: a conversation template object (fields of mlc-chat-config.json "conv_template").
// messages_json: OpenAI-style [{"role":..., "content": str | [{"type":"text","text":...}] | null}].
// A trailing generation prompt (assistant role with empty content) is appended unless the last
// message already is an assistant message with null content.
std::string RenderConversation(const std::string& conv_json, const std::string& messages_json);

}  // namespace mlcb
