// Minimal JSON helpers for the proxy: locate top-level members of an object without building a tree, and
// rewrite / insert / remove them in place.  Enough for the request surgery of the two-phase prefill/decode flow
// (the reference uses the jsmn tokenizer for the same job, ngx_http_prefill_module.c:106-291, 515-651).
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace omni_proxy {

struct JsonMember {
  std::string key;
  size_t key_begin = 0;     // position of the opening quote of the key
  size_t value_begin = 0;   // first character of the value
  size_t value_end = 0;     // one past the last character of the value
};

namespace detail {
inline size_t skip_ws(const std::string& s, size_t i) {
  while (i < s.size() && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) ++i;
  return i;
}
// returns one past the end of the string literal starting at s[i] == '"', or npos
inline size_t skip_string(const std::string& s, size_t i) {
  for (++i; i < s.size(); ++i) {
    if (s[i] == '\\') { ++i; continue; }
    if (s[i] == '"') return i + 1;
  }
  return std::string::npos;
}
// returns one past the end of the value starting at i, or npos on malformed input
inline size_t skip_value(const std::string& s, size_t i) {
  if (i >= s.size()) return std::string::npos;
  if (s[i] == '"') return skip_string(s, i);
  if (s[i] == '{' || s[i] == '[') {
    int depth = 0;
    for (; i < s.size(); ++i) {
      if (s[i] == '"') { i = skip_string(s, i); if (i == std::string::npos) return i; --i; continue; }
      if (s[i] == '{' || s[i] == '[') ++depth;
      else if (s[i] == '}' || s[i] == ']') { if (--depth == 0) return i + 1; }
    }
    return std::string::npos;
  }
  while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']' && s[i] != ' ' && s[i] != '\n' && s[i] != '\r' && s[i] != '\t') ++i;
  return i;
}
}  // namespace detail

// Top-level members of the object in `s`.  Returns false when `s` is not a JSON object.
inline bool json_members(const std::string& s, std::vector<JsonMember>& out) {
  out.clear();
  size_t i = detail::skip_ws(s, 0);
  if (i >= s.size() || s[i] != '{') return false;
  i = detail::skip_ws(s, i + 1);
  if (i < s.size() && s[i] == '}') return true;
  while (i < s.size()) {
    if (s[i] != '"') return false;
    JsonMember m;
    m.key_begin = i;
    size_t ke = detail::skip_string(s, i);
    if (ke == std::string::npos) return false;
    m.key = s.substr(i + 1, ke - i - 2);
    i = detail::skip_ws(s, ke);
    if (i >= s.size() || s[i] != ':') return false;
    i = detail::skip_ws(s, i + 1);
    m.value_begin = i;
    m.value_end = detail::skip_value(s, i);
    if (m.value_end == std::string::npos) return false;
    out.push_back(m);
    i = detail::skip_ws(s, m.value_end);
    if (i < s.size() && s[i] == ',') { i = detail::skip_ws(s, i + 1); continue; }
    if (i < s.size() && s[i] == '}') return true;
    return false;
  }
  return false;
}

inline bool json_get(const std::string& s, const std::string& key, std::string& value) {
  std::vector<JsonMember> ms;
  if (!json_members(s, ms)) return false;
  for (auto& m : ms)
    if (m.key == key) { value = s.substr(m.value_begin, m.value_end - m.value_begin); return true; }
  return false;
}

// Set (replace or append) a top-level member; `raw_value` is spliced verbatim.
inline bool json_set(std::string& s, const std::string& key, const std::string& raw_value) {
  std::vector<JsonMember> ms;
  if (!json_members(s, ms)) return false;
  for (auto& m : ms)
    if (m.key == key) { s.replace(m.value_begin, m.value_end - m.value_begin, raw_value); return true; }
  size_t close = s.rfind('}');
  if (close == std::string::npos) return false;
  std::string ins = (ms.empty() ? "" : ",") + std::string("\"") + key + "\":" + raw_value;
  s.insert(close, ins);
  return true;
}

inline bool json_remove(std::string& s, const std::string& key) {
  std::vector<JsonMember> ms;
  if (!json_members(s, ms)) return false;
  for (size_t k = 0; k < ms.size(); ++k) {
    if (ms[k].key != key) continue;
    size_t b = ms[k].key_begin, e = ms[k].value_end;
    if (k + 1 < ms.size()) e = ms[k + 1].key_begin;                 // swallow the following comma
    else if (k > 0) b = ms[k - 1].value_end;                        // or the preceding one
    s.erase(b, e - b);
    return true;
  }
  return true;
}

// first integer following `"name":` anywhere in a chunk of text (SSE body filters)
inline bool find_int_after(const std::string& s, const std::string& name, long long& out, size_t from = 0) {
  size_t p = s.rfind("\"" + name + "\"");
  if (p == std::string::npos || p < from) return false;
  p = s.find(':', p);
  if (p == std::string::npos) return false;
  ++p;
  while (p < s.size() && (s[p] == ' ')) ++p;
  if (p >= s.size() || !(s[p] == '-' || (s[p] >= '0' && s[p] <= '9'))) return false;
  out = atoll(s.c_str() + p);
  return true;
}

}  // namespace omni_proxy
