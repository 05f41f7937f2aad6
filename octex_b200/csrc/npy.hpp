// Memory-mapped .npy arrays and the small JSON reader of meta.json: the on-disk side of an index
// directory (format 1; layout described in docs/design.md:27-48 of hpdic/octex, read there by
// cpp/src/neighbors/octex/load.cu:215-313 and detail/npy.hpp:287-377).
#pragma once

#include "common.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cctype>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace octex_b200 {

// ---- JSON (objects, arrays, strings, numbers, true/false/null) -------------------------------

struct json_value {
  enum kind_t { null_k, bool_k, number_k, string_k, array_k, object_k } kind = null_k;
  double number = 0;
  bool boolean  = false;
  std::string text;
  std::vector<json_value> items;
  std::map<std::string, json_value> members;

  [[nodiscard]] auto has(std::string const& k) const -> bool
  {
    return kind == object_k && members.count(k) != 0;
  }
  [[nodiscard]] auto at(std::string const& k) const -> json_value const&
  {
    auto it = members.find(k);
    OCTEX_EXPECTS(kind == object_k && it != members.end(), "octex: meta.json lacks \"" + k + "\"");
    return it->second;
  }
  [[nodiscard]] auto num(std::string const& k, double fallback) const -> double
  {
    return has(k) && at(k).kind == number_k ? at(k).number : fallback;
  }
};

class json_reader {
 public:
  explicit json_reader(std::string const& s) : s_(s) {}
  auto parse() -> json_value
  {
    json_value v = value();
    skip();
    OCTEX_EXPECTS(at_ == s_.size(), "octex: trailing text in meta.json");
    return v;
  }

 private:
  std::string const& s_;
  size_t at_ = 0;

  void skip()
  {
    while (at_ < s_.size() && std::isspace(static_cast<unsigned char>(s_[at_])))
      at_++;
  }
  auto peek() -> char
  {
    skip();
    OCTEX_EXPECTS(at_ < s_.size(), "octex: meta.json ends early");
    return s_[at_];
  }
  void expect(char c)
  {
    OCTEX_EXPECTS(peek() == c, std::string("octex: meta.json: expected '") + c + "'");
    at_++;
  }
  auto string() -> std::string
  {
    expect('"');
    std::string out;
    while (true) {
      OCTEX_EXPECTS(at_ < s_.size(), "octex: meta.json: open string");
      char c = s_[at_++];
      if (c == '"') break;
      if (c == '\\') {
        OCTEX_EXPECTS(at_ < s_.size(), "octex: meta.json: open escape");
        char e = s_[at_++];
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            OCTEX_EXPECTS(at_ + 4 <= s_.size(), "octex: meta.json: short \\u escape");
            unsigned cp = static_cast<unsigned>(std::strtoul(s_.substr(at_, 4).c_str(), nullptr, 16));
            at_ += 4;
            if (cp < 0x80) {
              out += static_cast<char>(cp);
            } else if (cp < 0x800) {
              out += static_cast<char>(0xC0 | (cp >> 6));
              out += static_cast<char>(0x80 | (cp & 0x3F));
            } else {
              out += static_cast<char>(0xE0 | (cp >> 12));
              out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
              out += static_cast<char>(0x80 | (cp & 0x3F));
            }
            break;
          }
          default: out += e;
        }
      } else {
        out += c;
      }
    }
    return out;
  }
  auto value() -> json_value
  {
    json_value v;
    char c = peek();
    if (c == '{') {
      v.kind = json_value::object_k;
      at_++;
      if (peek() == '}') {
        at_++;
        return v;
      }
      while (true) {
        std::string k = string();
        expect(':');
        v.members[k] = value();
        if (peek() == ',') {
          at_++;
          continue;
        }
        expect('}');
        break;
      }
    } else if (c == '[') {
      v.kind = json_value::array_k;
      at_++;
      if (peek() == ']') {
        at_++;
        return v;
      }
      while (true) {
        v.items.push_back(value());
        if (peek() == ',') {
          at_++;
          continue;
        }
        expect(']');
        break;
      }
    } else if (c == '"') {
      v.kind = json_value::string_k;
      v.text = string();
    } else if (s_.compare(at_, 4, "true") == 0) {
      v.kind = json_value::bool_k, v.boolean = true, at_ += 4;
    } else if (s_.compare(at_, 5, "false") == 0) {
      v.kind = json_value::bool_k, at_ += 5;
    } else if (s_.compare(at_, 4, "null") == 0) {
      at_ += 4;
    } else {
      const char* b = s_.c_str() + at_;
      char* e       = nullptr;
      v.number      = std::strtod(b, &e);
      OCTEX_EXPECTS(e != b, "octex: meta.json: unexpected character");
      v.kind = json_value::number_k;
      at_ += static_cast<size_t>(e - b);
    }
    return v;
  }
};

inline auto read_text(std::string const& path) -> std::string
{
  std::ifstream f(path, std::ios::binary);
  OCTEX_EXPECTS(f.good(), "octex: cannot open " + path);
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

// ---- .npy ---------------------------------------------------------------------------------------

/// A read-only mapping of one .npy file (versions 1.0 - 3.0, little-endian, C order).
class npy_file {
 public:
  std::vector<int64_t> shape;
  std::string descr;  // e.g. "<f4"
  const char* data = nullptr;
  size_t bytes     = 0;

  explicit npy_file(std::string const& path)
  {
    fd_ = ::open(path.c_str(), O_RDONLY);
    OCTEX_EXPECTS(fd_ >= 0, "octex: cannot open " + path);
    struct stat st {};
    OCTEX_EXPECTS(::fstat(fd_, &st) == 0, "octex: cannot stat " + path);
    len_ = static_cast<size_t>(st.st_size);
    OCTEX_EXPECTS(len_ >= 10, "octex: " + path + " is not an .npy file");
    map_ = ::mmap(nullptr, len_, PROT_READ, MAP_PRIVATE, fd_, 0);
    OCTEX_EXPECTS(map_ != MAP_FAILED, "octex: cannot map " + path);
    auto* p = static_cast<const unsigned char*>(map_);
    OCTEX_EXPECTS(std::memcmp(p, "\x93NUMPY", 6) == 0, "octex: " + path + " is not an .npy file");
    const int major = p[6];
    size_t hlen = 0, hoff = 0;
    if (major == 1) {
      hlen = p[8] | (static_cast<size_t>(p[9]) << 8);
      hoff = 10;
    } else {
      OCTEX_EXPECTS(len_ >= 12, "octex: short .npy header in " + path);
      hlen = p[8] | (static_cast<size_t>(p[9]) << 8) | (static_cast<size_t>(p[10]) << 16) |
             (static_cast<size_t>(p[11]) << 24);
      hoff = 12;
    }
    OCTEX_EXPECTS(hoff + hlen <= len_, "octex: short .npy header in " + path);
    std::string h(reinterpret_cast<const char*>(p + hoff), hlen);
    descr = quoted_after(h, "'descr'", path);
    OCTEX_EXPECTS(h.find("'fortran_order': False") != std::string::npos,
                  "octex: " + path + " is not in C order");
    OCTEX_EXPECTS(descr.size() >= 2 && (descr[0] == '<' || descr[0] == '|'),
                  "octex: " + path + " is not little-endian");
    auto sp = h.find("'shape'");
    OCTEX_EXPECTS(sp != std::string::npos, "octex: no shape in " + path);
    auto lp = h.find('(', sp), rp = h.find(')', sp);
    OCTEX_EXPECTS(lp != std::string::npos && rp != std::string::npos && rp > lp,
                  "octex: bad shape in " + path);
    std::string dims = h.substr(lp + 1, rp - lp - 1);
    size_t i = 0;
    while (i < dims.size()) {
      while (i < dims.size() && !std::isdigit(static_cast<unsigned char>(dims[i])))
        i++;
      if (i >= dims.size()) break;
      size_t j = i;
      while (j < dims.size() && std::isdigit(static_cast<unsigned char>(dims[j])))
        j++;
      shape.push_back(std::strtoll(dims.substr(i, j - i).c_str(), nullptr, 10));
      i = j;
    }
    int64_t count = 1;
    for (auto d : shape)
      count *= d;
    const int item = std::atoi(descr.c_str() + 2);
    data           = reinterpret_cast<const char*>(p + hoff + hlen);
    bytes          = static_cast<size_t>(count) * static_cast<size_t>(item);
    OCTEX_EXPECTS(hoff + hlen + bytes <= len_, "octex: " + path + " is truncated");
  }
  npy_file(npy_file const&)                    = delete;
  auto operator=(npy_file const&) -> npy_file& = delete;
  ~npy_file()
  {
    if (map_ != nullptr && map_ != MAP_FAILED) ::munmap(map_, len_);
    if (fd_ >= 0) ::close(fd_);
  }
  void expect(std::string const& want, size_t rank, std::string const& name) const
  {
    OCTEX_EXPECTS(descr == want, "octex: " + name + ".npy holds " + descr + ", expected " + want);
    OCTEX_EXPECTS(shape.size() == rank, "octex: " + name + ".npy has the wrong rank");
  }
  template <typename T>
  [[nodiscard]] auto as() const -> const T*
  {
    return reinterpret_cast<const T*>(data);
  }

 private:
  int fd_     = -1;
  void* map_  = nullptr;
  size_t len_ = 0;

  static auto quoted_after(std::string const& h, std::string const& key, std::string const& path)
    -> std::string
  {
    auto k = h.find(key);
    OCTEX_EXPECTS(k != std::string::npos, "octex: no " + key + " in " + path);
    auto a = h.find('\'', k + key.size());
    OCTEX_EXPECTS(a != std::string::npos, "octex: bad header in " + path);
    auto b = h.find('\'', a + 1);
    OCTEX_EXPECTS(b != std::string::npos, "octex: bad header in " + path);
    return h.substr(a + 1, b - a - 1);
  }
};

}  // namespace octex_b200
