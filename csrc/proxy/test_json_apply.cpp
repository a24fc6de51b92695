// Applies the proxy's JSON member operations to documents given on standard input, for property tests that compare
// the result with a full JSON parser.  Input: records of four lines "op", "key", "raw value", "document" (every
// line hex-encoded so that any byte can appear).  Output per record: "1 <hex of the result>" or "0" when the helper
// refused the document.  Operations: get, set, remove, prefill (the body rewrite of the prefill phase).
#include <cstdio>
#include <iostream>
#include <string>

#include "json_min.h"

using namespace omni_proxy;

static std::string unhex(const std::string& h) {
  std::string out;
  for (size_t i = 0; i + 1 < h.size(); i += 2) out.push_back((char)std::stoi(h.substr(i, 2), nullptr, 16));
  return out;
}
static std::string hex(const std::string& s) {
  static const char* d = "0123456789abcdef";
  std::string out;
  for (unsigned char c : s) { out.push_back(d[c >> 4]); out.push_back(d[c & 15]); }
  return out;
}

int main() {
  std::string op, key, raw, doc;
  while (std::getline(std::cin, op) && std::getline(std::cin, key) && std::getline(std::cin, raw) && std::getline(std::cin, doc)) {
    op = unhex(op); key = unhex(key); raw = unhex(raw); doc = unhex(doc);
    bool ok = false;
    std::string out;
    if (op == "get") { ok = json_get(doc, key, out); }
    else if (op == "set") { ok = json_set(doc, key, raw); out = doc; }
    else if (op == "remove") { ok = json_remove(doc, key); out = doc; }
    else if (op == "prefill") {
      ok = json_set(doc, "max_tokens", "1") && json_set(doc, "stream", "false") && json_remove(doc, "stream_options");
      out = doc;
    }
    if (ok) printf("1 %s\n", hex(out).c_str()); else printf("0\n");
  }
  return 0;
}
