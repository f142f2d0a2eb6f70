#include "ir/xml.h"

#include <cctype>

namespace hl {
namespace xml {

namespace {
struct Cursor {
  const std::string& s;
  size_t i = 0;
  int line = 1;
  std::string err;
  explicit Cursor(const std::string& t) : s(t) {}
  bool eof() const { return i >= s.size(); }
  char peek(size_t k = 0) const { return i + k < s.size() ? s[i + k] : '\0'; }
  void adv(size_t k = 1) {
    for (size_t j = 0; j < k && i < s.size(); ++j, ++i)
      if (s[i] == '\n') ++line;
  }
  bool starts(const char* lit) const { return s.compare(i, std::char_traits<char>::length(lit), lit) == 0; }
  void skipWs() {
    while (!eof() && std::isspace((unsigned char)s[i])) adv();
  }
  bool fail(const std::string& what) {
    if (err.empty()) err = "line " + std::to_string(line) + ": " + what;
    return false;
  }
};

bool nameChar(char c) { return std::isalnum((unsigned char)c) || c == '_' || c == '-' || c == ':' || c == '.'; }

std::string decode(const std::string& raw) {
  std::string out;
  out.reserve(raw.size());
  for (size_t i = 0; i < raw.size(); ++i) {
    if (raw[i] != '&') {
      out.push_back(raw[i]);
      continue;
    }
    static const struct { const char* ent; char c; } table[] = {
        {"&amp;", '&'}, {"&lt;", '<'}, {"&gt;", '>'}, {"&quot;", '"'}, {"&apos;", '\''}};
    bool hit = false;
    for (auto& e : table) {
      size_t n = std::char_traits<char>::length(e.ent);
      if (raw.compare(i, n, e.ent) == 0) {
        out.push_back(e.c);
        i += n - 1;
        hit = true;
        break;
      }
    }
    if (!hit) out.push_back('&');
  }
  return out;
}

bool skipMisc(Cursor& c) {
  for (;;) {
    c.skipWs();
    if (c.starts("<!--")) {
      size_t end = c.s.find("-->", c.i + 4);
      if (end == std::string::npos) return c.fail("unterminated comment");
      c.adv(end + 3 - c.i);
    } else if (c.starts("<?")) {
      size_t end = c.s.find("?>", c.i + 2);
      if (end == std::string::npos) return c.fail("unterminated declaration");
      c.adv(end + 2 - c.i);
    } else if (c.starts("<!")) {
      size_t end = c.s.find('>', c.i);
      if (end == std::string::npos) return c.fail("unterminated <! section");
      c.adv(end + 1 - c.i);
    } else {
      return true;
    }
  }
}

std::unique_ptr<Node> parseElement(Cursor& c, int depth) {
  if (depth > 64) {
    c.fail("nesting too deep");
    return nullptr;
  }
  if (c.peek() != '<') {
    c.fail("expected '<'");
    return nullptr;
  }
  std::unique_ptr<Node> n(new Node());
  n->line = c.line;
  c.adv();
  while (nameChar(c.peek())) {
    n->name.push_back(c.peek());
    c.adv();
  }
  if (n->name.empty()) {
    c.fail("element without a name");
    return nullptr;
  }
  for (;;) {
    c.skipWs();
    if (c.eof()) {
      c.fail("unexpected end inside <" + n->name + ">");
      return nullptr;
    }
    if (c.starts("/>")) {
      c.adv(2);
      return n;
    }
    if (c.peek() == '>') {
      c.adv();
      break;
    }
    std::string key;
    while (nameChar(c.peek())) {
      key.push_back(c.peek());
      c.adv();
    }
    if (key.empty()) {
      c.fail("bad attribute in <" + n->name + ">");
      return nullptr;
    }
    c.skipWs();
    if (c.peek() != '=') {
      c.fail("attribute '" + key + "' without a value");
      return nullptr;
    }
    c.adv();
    c.skipWs();
    const char q = c.peek();
    if (q != '"' && q != '\'') {
      c.fail("attribute '" + key + "' value must be quoted");
      return nullptr;
    }
    c.adv();
    size_t end = c.s.find(q, c.i);
    if (end == std::string::npos) {
      c.fail("unterminated attribute value");
      return nullptr;
    }
    n->attrs[key] = decode(c.s.substr(c.i, end - c.i));
    c.adv(end + 1 - c.i);
  }
  // content
  for (;;) {
    if (c.eof()) {
      c.fail("missing </" + n->name + ">");
      return nullptr;
    }
    if (c.starts("<!--")) {
      size_t end = c.s.find("-->", c.i + 4);
      if (end == std::string::npos) {
        c.fail("unterminated comment");
        return nullptr;
      }
      c.adv(end + 3 - c.i);
    } else if (c.starts("<![CDATA[")) {
      size_t end = c.s.find("]]>", c.i);
      if (end == std::string::npos) {
        c.fail("unterminated CDATA");
        return nullptr;
      }
      n->text += c.s.substr(c.i + 9, end - c.i - 9);
      c.adv(end + 3 - c.i);
    } else if (c.starts("</")) {
      c.adv(2);
      std::string close;
      while (nameChar(c.peek())) {
        close.push_back(c.peek());
        c.adv();
      }
      c.skipWs();
      if (c.peek() != '>' || close != n->name) {
        c.fail("mismatched closing tag </" + close + "> for <" + n->name + ">");
        return nullptr;
      }
      c.adv();
      return n;
    } else if (c.peek() == '<') {
      auto child = parseElement(c, depth + 1);
      if (!child) return nullptr;
      n->children.push_back(std::move(child));
    } else {
      size_t end = c.s.find('<', c.i);
      if (end == std::string::npos) end = c.s.size();
      n->text += decode(c.s.substr(c.i, end - c.i));
      c.adv(end - c.i);
    }
  }
}
}  // namespace

std::unique_ptr<Node> parse(const std::string& text, std::string* error) {
  Cursor c(text);
  if (!skipMisc(c)) {
    if (error) *error = c.err;
    return nullptr;
  }
  if (c.eof()) {
    if (error) *error = "empty document";
    return nullptr;
  }
  auto root = parseElement(c, 0);
  if (!root) {
    if (error) *error = c.err;
    return nullptr;
  }
  if (!skipMisc(c) || !c.eof()) {
    if (error) *error = c.err.empty() ? ("line " + std::to_string(c.line) + ": content after the root element") : c.err;
    return nullptr;
  }
  return root;
}

}  // namespace xml
}  // namespace hl
