// A small reader for protobuf *text format* ("key: value", "key { ... }",
// repeated fields, '#' comments, "[pkg.ext]" extension names), which is how the
// reference's applications are configured (app/linear_method/proto/linear.proto,
// example/linear/*/*.conf). The result is a generic tree.
#pragma once
#include "common.h"

namespace PS {

struct TextNode {
  // scalar fields and sub-messages in file order; a name may repeat
  std::vector<std::pair<std::string, std::string>> scalars;
  std::vector<std::pair<std::string, TextNode>> children;

  bool has(const std::string& k) const {
    for (auto& s : scalars) if (s.first == k) return true;
    for (auto& c : children) if (c.first == k) return true;
    return false;
  }
  std::string str(const std::string& k, const std::string& def = "") const {
    for (auto& s : scalars) if (s.first == k) return s.second;
    return def;
  }
  double num(const std::string& k, double def = 0) const {
    for (auto& s : scalars) if (s.first == k) return atof(s.second.c_str());
    return def;
  }
  long long integer(const std::string& k, long long def = 0) const {
    for (auto& s : scalars) if (s.first == k) return atoll(s.second.c_str());
    return def;
  }
  bool boolean(const std::string& k, bool def = false) const {
    for (auto& s : scalars) if (s.first == k) return s.second == "true" || s.second == "1";
    return def;
  }
  std::vector<std::string> all(const std::string& k) const {
    std::vector<std::string> out;
    for (auto& s : scalars) if (s.first == k) out.push_back(s.second);
    return out;
  }
  const TextNode* child(const std::string& k) const {
    for (auto& c : children) if (c.first == k) return &c.second;
    return nullptr;
  }
  std::vector<const TextNode*> children_of(const std::string& k) const {
    std::vector<const TextNode*> out;
    for (auto& c : children) if (c.first == k) out.push_back(&c.second);
    return out;
  }
};

class TextProtoParser {
 public:
  static TextNode Parse(const std::string& text) {
    TextProtoParser p(text);
    TextNode root;
    p.ParseBody(&root, false);
    return root;
  }
 private:
  explicit TextProtoParser(const std::string& t) : s_(t) {}
  void SkipSpace() {
    while (i_ < s_.size()) {
      char c = s_[i_];
      if (c == '#') { while (i_ < s_.size() && s_[i_] != '\n') ++i_; }
      else if (isspace((unsigned char)c) || c == ',' || c == ';') ++i_;
      else break;
    }
  }
  std::string Name() {
    SkipSpace();
    std::string n;
    if (i_ < s_.size() && s_[i_] == '[') {        // extension: keep the last component
      size_t e = s_.find(']', i_);
      PS_CHECK(e != std::string::npos) << "unterminated [extension] name";
      std::string full = s_.substr(i_ + 1, e - i_ - 1);
      size_t dot = full.find_last_of('.');
      n = dot == std::string::npos ? full : full.substr(dot + 1);
      i_ = e + 1;
      return n;
    }
    while (i_ < s_.size() && (isalnum((unsigned char)s_[i_]) || s_[i_] == '_' || s_[i_] == '.')) n.push_back(s_[i_++]);
    return n;
  }
  std::string Value() {
    SkipSpace();
    std::string v;
    if (i_ < s_.size() && (s_[i_] == '"' || s_[i_] == '\'')) {
      char q = s_[i_++];
      while (i_ < s_.size() && s_[i_] != q) {
        if (s_[i_] == '\\' && i_ + 1 < s_.size()) {
          char c = s_[++i_];
          v.push_back(c == 'n' ? '\n' : c == 't' ? '\t' : c);
          ++i_;
        } else v.push_back(s_[i_++]);
      }
      PS_CHECK_LT(i_, s_.size()) << "unterminated string";
      ++i_;
      return v;
    }
    while (i_ < s_.size() && !isspace((unsigned char)s_[i_]) && s_[i_] != '}' && s_[i_] != '#' && s_[i_] != ',' && s_[i_] != ';')
      v.push_back(s_[i_++]);
    return v;
  }
  void ParseBody(TextNode* node, bool nested) {
    while (true) {
      SkipSpace();
      if (i_ >= s_.size()) { PS_CHECK(!nested) << "missing '}'"; return; }
      if (s_[i_] == '}') { PS_CHECK(nested) << "unexpected '}'"; ++i_; return; }
      std::string name = Name();
      PS_CHECK(!name.empty()) << "parse error near offset " << i_ << ": '" << s_.substr(i_, 20) << "'";
      SkipSpace();
      bool colon = false;
      if (i_ < s_.size() && s_[i_] == ':') { colon = true; ++i_; SkipSpace(); }
      if (i_ < s_.size() && (s_[i_] == '{' || s_[i_] == '<')) {
        ++i_;
        node->children.emplace_back(name, TextNode());
        ParseBody(&node->children.back().second, true);
      } else {
        PS_CHECK(colon) << "expected ':' after " << name;
        node->scalars.emplace_back(name, Value());
      }
    }
  }
  const std::string& s_;
  size_t i_ = 0;
};

}  // namespace PS
