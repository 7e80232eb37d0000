#include "tokenizer.hpp"

#include <algorithm>
#include <climits>
#include <cstdio>
#include <stdexcept>

namespace pk {
namespace {

void append_utf8(std::string& s, uint32_t cp) {
  if (cp < 0x80) {
    s.push_back((char)cp);
  } else if (cp < 0x800) {
    s.push_back((char)(0xC0 | (cp >> 6)));
    s.push_back((char)(0x80 | (cp & 0x3F)));
  } else if (cp < 0x10000) {
    s.push_back((char)(0xE0 | (cp >> 12)));
    s.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
    s.push_back((char)(0x80 | (cp & 0x3F)));
  } else {
    s.push_back((char)(0xF0 | (cp >> 18)));
    s.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
    s.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
    s.push_back((char)(0x80 | (cp & 0x3F)));
  }
}

// Next code point of a UTF-8 string; advances i. Malformed bytes come back as themselves.
uint32_t next_cp(const std::string& s, size_t& i) {
  const unsigned char c = (unsigned char)s[i];
  int len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
  if (i + (size_t)len > s.size()) len = 1;
  uint32_t cp = len == 1 ? c : c & (0xFF >> (len + 1));
  for (int k = 1; k < len; ++k) cp = (cp << 6) | ((unsigned char)s[i + k] & 0x3F);
  i += (size_t)len;
  return cp;
}

bool is_space(unsigned char c) { return c == ' ' || (c >= 9 && c <= 13); }
bool is_letter(unsigned char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c >= 0x80; }
bool is_digit(unsigned char c) { return c >= '0' && c <= '9'; }
bool is_other(unsigned char c) { return !is_space(c) && !is_letter(c) && !is_digit(c); }

}  // namespace

BpeTokenizer::BpeTokenizer(std::vector<std::string> tokens, const std::vector<std::string>& merges, const std::vector<int>& special)
    : tokens_(std::move(tokens)) {
  // GPT-2 byte <-> unicode table: printable bytes map to themselves, the rest to 256 + n
  std::vector<int> printable;
  for (int b = '!'; b <= '~'; ++b) printable.push_back(b);
  for (int b = 0xA1; b <= 0xAC; ++b) printable.push_back(b);
  for (int b = 0xAE; b <= 0xFF; ++b) printable.push_back(b);
  std::vector<bool> is_print(256, false);
  for (int b : printable) is_print[b] = true;
  int extra = 0;
  for (int b = 0; b < 256; ++b) {
    const uint32_t cp = is_print[b] ? (uint32_t)b : 256u + (uint32_t)extra++;
    append_utf8(byte_to_piece_[b], cp);
    cp_to_byte_[cp] = (uint8_t)b;
  }
  for (size_t i = 0; i < tokens_.size(); ++i) vocab_.emplace(tokens_[i], (int)i);
  int r = 0;
  for (const std::string& m : merges) {
    const size_t sp = m.find(' ');
    if (sp == std::string::npos) continue;
    rank_.emplace(m.substr(0, sp) + '\x01' + m.substr(sp + 1), r++);
  }
  is_special_.assign(tokens_.size(), false);
  for (int id : special) {
    if (id < 0 || id >= (int)tokens_.size() || tokens_[id].empty()) continue;
    is_special_[id] = true;
    special_.emplace_back(tokens_[id], id);
  }
  std::sort(special_.begin(), special_.end(), [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });
}

BpeTokenizer BpeTokenizer::from_gguf(const GgufFile& file) {
  const Json& md = file.metadata();
  const Json* toks = md.find("tokenizer.ggml.tokens");
  if (toks == nullptr || !toks->is_array()) throw std::runtime_error("tokenizer: GGUF has no tokenizer.ggml.tokens");
  const std::string model = md.get_string("tokenizer.ggml.model", "gpt2");
  if (model != "gpt2" && model != "bpe") throw std::runtime_error("tokenizer: unsupported tokenizer model " + model);
  std::vector<std::string> tokens, merges;
  for (const Json& t : toks->items()) tokens.push_back(t.as_string());
  if (const Json* m = md.find("tokenizer.ggml.merges"))
    for (const Json& x : m->items()) merges.push_back(x.as_string());
  std::vector<int> special;
  if (const Json* ty = md.find("tokenizer.ggml.token_type")) {
    int i = 0;
    for (const Json& x : ty->items()) {
      const int64_t v = x.as_int();
      if (v == 3 || v == 4) special.push_back(i);   // control, user defined
      ++i;
    }
  }
  return BpeTokenizer(std::move(tokens), merges, special);
}

BpeTokenizer BpeTokenizer::from_hf_dir(const std::string& dir_or_file) {
  std::string path = dir_or_file;
  const std::string suffix = ".json";
  if (path.size() < suffix.size() || path.compare(path.size() - suffix.size(), suffix.size(), suffix) != 0) path += "/tokenizer.json";
  FILE* f = std::fopen(path.c_str(), "rb");
  if (f == nullptr) throw std::runtime_error("tokenizer: cannot open " + path);
  std::string text;
  char buf[1 << 16];
  size_t got;
  while ((got = std::fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, got);
  std::fclose(f);
  const Json root = Json::parse(text);
  const Json* model = root.find("model");
  if (model == nullptr || !model->is_object()) throw std::runtime_error("tokenizer: " + path + " has no model section");
  const std::string type = model->get_string("type", "BPE");
  if (type != "BPE") throw std::runtime_error("tokenizer: unsupported model type " + type + " (byte-level BPE only)");
  const Json* vocab = model->find("vocab");
  if (vocab == nullptr || !vocab->is_object()) throw std::runtime_error("tokenizer: model.vocab is missing");
  int64_t max_id = -1;
  for (const auto& kv : vocab->members()) max_id = std::max<int64_t>(max_id, kv.second.as_int());
  const Json* added = root.find("added_tokens");
  if (added != nullptr && added->is_array())
    for (const Json& a : added->items()) max_id = std::max<int64_t>(max_id, a.get_int("id", -1));
  if (max_id < 0 || max_id > (1 << 24)) throw std::runtime_error("tokenizer: implausible vocabulary size");
  std::vector<std::string> tokens((size_t)max_id + 1);
  for (const auto& kv : vocab->members()) {
    const int64_t id = kv.second.as_int();
    if (id < 0) throw std::runtime_error("tokenizer: negative token id");
    tokens[(size_t)id] = kv.first;
  }
  std::vector<int> special;
  if (added != nullptr && added->is_array())
    for (const Json& a : added->items()) {
      const int64_t id = a.get_int("id", -1);
      if (id < 0) continue;
      tokens[(size_t)id] = a.get_string("content", tokens[(size_t)id]);
      special.push_back((int)id);   // added tokens are matched verbatim, whether flagged special or not
    }
  std::vector<std::string> merges;
  if (const Json* m = model->find("merges"))
    for (const Json& x : m->items()) {
      if (x.is_string()) merges.push_back(x.as_string());
      else if (x.is_array() && x.size() == 2) merges.push_back(x.items()[0].as_string() + " " + x.items()[1].as_string());
    }
  return BpeTokenizer(std::move(tokens), merges, special);
}

int BpeTokenizer::token_id(const std::string& piece) const {
  auto it = vocab_.find(piece);
  return it == vocab_.end() ? -1 : it->second;
}

std::vector<std::string> BpeTokenizer::pre_tokenize(const std::string& s) {
  std::vector<std::string> out;
  const size_t n = s.size();
  size_t i = 0;
  auto at = [&](size_t k) -> unsigned char { return k < n ? (unsigned char)s[k] : 0; };
  while (i < n) {
    const unsigned char c = at(i);
    if (c == '\'') {
      const unsigned char a = at(i + 1), b = at(i + 2);
      size_t len = 0;
      if (i + 2 < n + 0 && ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) && i + 2 < n) len = 3;
      else if (i + 1 < n && (a == 's' || a == 't' || a == 'm' || a == 'd')) len = 2;
      if (len) {
        out.push_back(s.substr(i, len));
        i += len;
        continue;
      }
    }
    size_t j = i + ((c == ' ' && i + 1 < n && !is_space(at(i + 1))) ? 1 : 0);
    if (j < n && !is_space(at(j))) {
      const unsigned char f = at(j);
      size_t k = j;
      if (is_letter(f)) while (k < n && is_letter(at(k))) ++k;
      else if (is_digit(f)) while (k < n && is_digit(at(k))) ++k;
      else while (k < n && is_other(at(k))) ++k;
      out.push_back(s.substr(i, k - i));
      i = k;
      continue;
    }
    // whitespace run: all of it at the end of the text, otherwise all but the last character (which joins the next
    // piece when it is a space, or stands alone)
    size_t k = i;
    while (k < n && is_space(at(k))) ++k;
    size_t len = k - i;
    if (k < n && len > 1) len -= 1;
    out.push_back(s.substr(i, len));
    i += len;
  }
  return out;
}

void BpeTokenizer::bpe(const std::string& word, std::vector<int>& out) const {
  std::vector<std::string> sym;
  for (unsigned char c : word) sym.push_back(byte_to_piece_[c]);
  while (sym.size() > 1) {
    int best = INT_MAX;
    size_t where = 0;
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      auto it = rank_.find(sym[i] + '\x01' + sym[i + 1]);
      if (it != rank_.end() && it->second < best) {
        best = it->second;
        where = i;
      }
    }
    if (best == INT_MAX) break;
    // merge every occurrence of the best pair, left to right
    const std::string a = sym[where], b = sym[where + 1];
    std::vector<std::string> next;
    for (size_t i = 0; i < sym.size();) {
      if (i + 1 < sym.size() && sym[i] == a && sym[i + 1] == b) {
        next.push_back(a + b);
        i += 2;
      } else {
        next.push_back(sym[i]);
        i += 1;
      }
    }
    sym.swap(next);
  }
  for (const std::string& p : sym) {
    auto it = vocab_.find(p);
    if (it != vocab_.end()) {
      out.push_back(it->second);
    } else {
      // not in the vocabulary as a whole: fall back to its bytes' single-symbol tokens
      size_t i = 0;
      while (i < p.size()) {
        const size_t start = i;
        next_cp(p, i);
        auto one = vocab_.find(p.substr(start, i - start));
        if (one != vocab_.end()) out.push_back(one->second);
      }
    }
  }
}

std::vector<int> BpeTokenizer::encode(const std::string& text, bool parse_special) const {
  std::vector<int> out;
  size_t i = 0;
  std::string plain;
  auto flush = [&] {
    for (const std::string& w : pre_tokenize(plain)) bpe(w, out);
    plain.clear();
  };
  while (i < text.size()) {
    bool matched = false;
    if (parse_special) {
      for (const auto& sp : special_) {
        if (text.compare(i, sp.first.size(), sp.first) == 0) {
          flush();
          out.push_back(sp.second);
          i += sp.first.size();
          matched = true;
          break;
        }
      }
    }
    if (!matched) plain.push_back(text[i++]);
  }
  flush();
  return out;
}

std::string BpeTokenizer::decode(const std::vector<int>& ids, bool skip_special) const {
  std::string out;
  for (int id : ids) {
    if (id < 0 || id >= (int)tokens_.size()) continue;
    if (is_special_[id]) {
      if (!skip_special) out += tokens_[id];
      continue;
    }
    const std::string& p = tokens_[id];
    size_t i = 0;
    while (i < p.size()) {
      const uint32_t cp = next_cp(p, i);
      auto it = cp_to_byte_.find(cp);
      if (it != cp_to_byte_.end()) out.push_back((char)it->second);
      else append_utf8(out, cp);
    }
  }
  return out;
}

}  // namespace pk
