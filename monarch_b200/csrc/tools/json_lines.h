// JSON lines of the allocator protocol: a small reader (objects, arrays, strings, numbers,
// booleans, null) and string quoting that keeps the output valid UTF-8.  Shared by the daemon
// (process_allocator.cpp) and the client stub (remote_exec.cpp).
#pragma once

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace mbtools {

struct Json {
  enum Kind { Null, Bool, Num, Str, Obj, Arr } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::map<std::string, Json> obj;
  std::vector<Json> arr;
  const Json* get(const std::string& k) const {
    auto it = obj.find(k);
    return it == obj.end() ? nullptr : &it->second;
  }
  bool truthy() const {
    switch (kind) {
      case Null: return false;
      case Bool: return b;
      case Num: return num != 0;
      case Str: return !str.empty();
      case Obj: return !obj.empty();
      case Arr: return !arr.empty();
    }
    return false;
  }
};

struct Parser {
  const std::string& s;
  size_t i = 0;
  bool ok = true;
  explicit Parser(const std::string& t) : s(t) {}
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) ++i;
  }
  static void utf8(std::string& out, unsigned cp) {
    if (cp < 0x80) {
      out += (char)cp;
    } else if (cp < 0x800) {
      out += (char)(0xC0 | (cp >> 6));
      out += (char)(0x80 | (cp & 0x3F));
    } else if (cp < 0x10000) {
      out += (char)(0xE0 | (cp >> 12));
      out += (char)(0x80 | ((cp >> 6) & 0x3F));
      out += (char)(0x80 | (cp & 0x3F));
    } else {
      out += (char)(0xF0 | (cp >> 18));
      out += (char)(0x80 | ((cp >> 12) & 0x3F));
      out += (char)(0x80 | ((cp >> 6) & 0x3F));
      out += (char)(0x80 | (cp & 0x3F));
    }
  }
  bool hex4(unsigned& v) {
    if (i + 4 > s.size()) return false;
    v = 0;
    for (int k = 0; k < 4; ++k) {
      char c = s[i++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
      else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
      else return false;
    }
    return true;
  }
  std::string string() {
    std::string out;
    ++i;  // opening quote
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c != '\\') {
        out += c;
        continue;
      }
      if (i >= s.size()) { ok = false; return out; }
      char e = s[i++];
      switch (e) {
        case 'n': out += '\n'; break;
        case 't': out += '\t'; break;
        case 'r': out += '\r'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'u': {
          unsigned cp = 0;
          if (!hex4(cp)) { ok = false; return out; }
          if (cp >= 0xD800 && cp < 0xDC00 && i + 1 < s.size() && s[i] == '\\' && s[i + 1] == 'u') {
            i += 2;
            unsigned lo = 0;
            if (!hex4(lo)) { ok = false; return out; }
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(out, cp);
          break;
        }
        default: out += e;
      }
    }
    if (i >= s.size()) ok = false; else ++i;
    return out;
  }
  Json value(int depth = 0) {
    Json j;
    ws();
    if (i >= s.size() || depth > 32) { ok = false; return j; }
    char c = s[i];
    if (c == '{') {
      j.kind = Json::Obj;
      ++i;
      ws();
      if (i < s.size() && s[i] == '}') { ++i; return j; }
      while (ok) {
        ws();
        if (i >= s.size() || s[i] != '"') { ok = false; break; }
        std::string k = string();
        ws();
        if (i >= s.size() || s[i] != ':') { ok = false; break; }
        ++i;
        j.obj[k] = value(depth + 1);
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == '}') { ++i; break; }
        ok = false;
      }
    } else if (c == '[') {
      j.kind = Json::Arr;
      ++i;
      ws();
      if (i < s.size() && s[i] == ']') { ++i; return j; }
      while (ok) {
        j.arr.push_back(value(depth + 1));
        ws();
        if (i < s.size() && s[i] == ',') { ++i; continue; }
        if (i < s.size() && s[i] == ']') { ++i; break; }
        ok = false;
      }
    } else if (c == '"') {
      j.kind = Json::Str;
      j.str = string();
    } else if (s.compare(i, 4, "true") == 0) {
      j.kind = Json::Bool; j.b = true; i += 4;
    } else if (s.compare(i, 5, "false") == 0) {
      j.kind = Json::Bool; i += 5;
    } else if (s.compare(i, 4, "null") == 0) {
      i += 4;
    } else {
      char* end = nullptr;
      j.num = std::strtod(s.c_str() + i, &end);
      if (end == s.c_str() + i) { ok = false; return j; }
      j.kind = Json::Num;
      i = (size_t)(end - s.c_str());
    }
    return j;
  }
};

// Length of the well-formed UTF-8 sequence that starts at t[i], or 0.
inline size_t utf8_len(const std::string& t, size_t i) {
  const unsigned char c = (unsigned char)t[i];
  size_t n = c >= 0xF0 && c <= 0xF4 ? 4 : c >= 0xE0 ? 3 : c >= 0xC2 && c < 0xE0 ? 2 : 0;
  if (n == 0 || i + n > t.size()) return 0;
  for (size_t k = 1; k < n; ++k)
    if (((unsigned char)t[i + k] & 0xC0) != 0x80) return 0;
  return n;
}

inline std::string quote(const std::string& t) {
  std::string out = "\"";
  char buf[8];
  for (size_t i = 0; i < t.size(); ++i) {
    const unsigned char c = (unsigned char)t[i];
    if (c >= 0x80) {                 // the child's output need not be text
      const size_t n = utf8_len(t, i);
      if (n == 0) {
        out += "\\ufffd";
      } else {
        out.append(t, i, n);
        i += n - 1;
      }
      continue;
    }
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          std::snprintf(buf, sizeof buf, "\\u%04x", c);
          out += buf;
        } else {
          out += (char)c;
        }
    }
  }
  return out + "\"";
}


// Environment variables a client may set for the procs it asks for.
inline bool env_allowed(const std::string& k) {
  static const char* kAllowPrefix[] = {"HYPERACTOR_", "MONARCH_", "MB200_", "MASTER_"};
  static const char* kAllowExact[] = {"CUDA_VISIBLE_DEVICES", "LOCAL_RANK", "RANK", "WORLD_SIZE",
                                      "PYTHONPATH"};
  if (k == "MB200_ALLOCATOR_TOKEN") return false;
  for (const char* p : kAllowPrefix)
    if (k.compare(0, std::strlen(p), p) == 0) return true;
  for (const char* e : kAllowExact)
    if (k == e) return true;
  return false;
}

}  // namespace mbtools
