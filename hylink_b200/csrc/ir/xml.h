// A small non-validating XML reader: elements, attributes, comments, the XML
// declaration, character data and the five predefined entities. Enough for
// schedule files; no DTDs, namespaces or processing instructions beyond <?xml?>.
//
// Parity: the reference vendors tinyxml2 for the same job
// (pcie-ccl-cuda/src/third_party/tinyxml2, used by src/ir/ir_loader.cpp:16-79).
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace hl {
namespace xml {

struct Node {
  std::string name;
  std::map<std::string, std::string> attrs;
  std::vector<std::unique_ptr<Node>> children;
  std::string text;
  int line = 0;
  const std::string* attr(const std::string& k) const {
    auto it = attrs.find(k);
    return it == attrs.end() ? nullptr : &it->second;
  }
};

// Returns the root element, or nullptr with *error set ("line N: what").
std::unique_ptr<Node> parse(const std::string& text, std::string* error);

}  // namespace xml
}  // namespace hl
