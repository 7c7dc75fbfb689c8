#include "conv_template.h"

#include <stdexcept>
#include <vector>

#include "json.h"

namespace mlcb {

namespace {
std::string ReplaceAll(std::string s, const std::string& from, const std::string& to) {
  if (from.empty()) return s;
  size_t pos = 0;
  while ((pos = s.find(from, pos)) != std::string::npos) {
    s.replace(pos, from.size(), to);
    pos += to.size();
  }
  return s;
}
std::string Placeholder(const std::string& role) {
  if (role == "system") return "{system_message}";
  if (role == "user") return "{user_message}";
  if (role == "assistant") return "{assistant_message}";
  if (role == "tool") return "{tool_message}";
  return "{" + role + "_message}";
}
}  // namespace

const char* const kImagePlaceholder = "\x02<|mlcb-image|>\x03";

std::string RenderConversation(const std::string& conv_json, const std::string& messages_json,
                               std::vector<std::string>* image_urls) {
  json::Value cv = json::parse(conv_json);
  json::Value mv = json::parse(messages_json);
  const json::Object& c = cv.as_object();
  const std::string system_template = json::get_or<std::string>(c, "system_template", "{system_message}");
  std::string system_message = json::get_or<std::string>(c, "system_message", "");
  const bool add_role_after_system = json::get_or<bool>(c, "add_role_after_system_message", true);
  const std::string role_content_sep = json::get_or<std::string>(c, "role_content_sep", "");
  const std::string role_empty_sep = json::get_or<std::string>(c, "role_empty_sep", "");
  const std::string function_string = json::get_or<std::string>(c, "function_string", "");
  std::vector<std::string> seps;
  if (auto* s = c.find("seps"); s && s->is_array())
    for (auto& e : s->as_array()) seps.push_back(e.as_string());
  if (seps.empty() || seps.size() > 2) throw std::runtime_error("seps should have size 1 or 2.");
  if (seps.size() == 1) seps.push_back(seps[0]);
  const json::Object* roles = nullptr;
  if (auto* r = c.find("roles"); r && r->is_object()) roles = &r->as_object();
  if (!roles) throw std::runtime_error("conversation template has no roles");
  auto role_template = [&](const std::string& role) {
    if (auto* rt = c.find("role_templates"); rt && rt->is_object())
      if (auto* v = rt->as_object().find(role); v && v->is_string()) return v->as_string();
    return Placeholder(role);
  };

  // collect (role, content) pairs; a leading system message overrides the template's
  struct Msg { std::string role; bool has_content; std::string content; };
  std::vector<Msg> msgs;
  bool first = true;
  for (auto& m : mv.as_array()) {
    const json::Object& mo = m.as_object();
    std::string role = json::get_or<std::string>(mo, "role", "");
    std::string text;
    bool has = false;
    if (auto* ct = mo.find("content"); ct) {
      if (ct->is_string()) {
        text = ct->as_string();
        has = true;
      } else if (ct->is_array()) {
        for (auto& part : ct->as_array()) {
          const json::Object& po = part.as_object();
          const std::string type = json::get_or<std::string>(po, "type", "");
          if (type == "text") {
            text += json::get_or<std::string>(po, "text", "");
          } else if (type == "image_url" && image_urls != nullptr) {
            const json::Value* iu = po.find("image_url");
            std::string url;
            if (iu && iu->is_string()) url = iu->as_string();
            else if (iu && iu->is_object()) url = json::get_or<std::string>(iu->as_object(), "url", "");
            if (url.empty()) throw std::runtime_error("an image_url content part needs a url");
            image_urls->push_back(url);
            text += kImagePlaceholder;
            text += "\n";  // an image is followed by a newline, as in the Python renderer
          } else {
            throw std::runtime_error("unsupported content part type \"" + type + "\"");
          }
        }
        has = true;
      }
    }
    if (role == "system") {
      if (!first) throw std::runtime_error("System prompt at position other than the beginning is not supported.");
      system_message = text;
    } else {
      msgs.push_back({role, has, text});
    }
    first = false;
  }
  if (msgs.empty() || msgs.back().role != "assistant" || msgs.back().has_content)
    msgs.push_back({"assistant", false, ""});

  std::string out;
  const std::string system_msg = ReplaceAll(system_template, "{system_message}", system_message);
  out += system_msg;
  for (size_t i = 0; i < msgs.size(); ++i) {
    const Msg& m = msgs[i];
    auto* rn = roles->find(m.role);
    if (!rn) throw std::runtime_error("Role \"" + m.role + "\" is not a supported role");
    const std::string& role_name = rn->as_string();
    const std::string& sep = m.role == "assistant" ? seps[1] : seps[0];
    if (!m.has_content) {
      out += role_name + role_empty_sep;
      continue;
    }
    const bool skip_prefix = !add_role_after_system && !system_msg.empty() && i == 0;
    if (!skip_prefix) out += role_name + role_content_sep;
    out += ReplaceAll(role_template(m.role), Placeholder(m.role), m.content);
    out += sep;
  }
  // the last function-string placeholder receives the tool description, the others vanish
  const std::string fph = "{function_string}";
  size_t last = out.rfind(fph);
  if (last != std::string::npos) out.replace(last, fph.size(), function_string);
  out = ReplaceAll(out, fph, "");
  return out;
}

}  // namespace mlcb
