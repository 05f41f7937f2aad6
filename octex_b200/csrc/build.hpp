// The index builder's interface inside the library (the public one is octex_b200::build in
// include/octex_b200.hpp and cuvsOctexBuild in include/octex_b200.h).
#pragma once

#include "common.hpp"

#include <octex_b200.hpp>

#include <string>
#include <sys/stat.h>

namespace octex_b200 {

/// Creates the directory (and its parents) when it does not exist.
inline void make_directory(std::string const& path)
{
  std::string at;
  for (size_t i = 0; i <= path.size(); i++) {
    if (i == path.size() || path[i] == '/') {
      if (!at.empty() && at != "/") {
        if (::mkdir(at.c_str(), 0777) != 0 && errno != EEXIST) throw error("octex: cannot create " + at);
      }
    }
    if (i < path.size()) at.push_back(path[i]);
  }
  struct stat st {};
  OCTEX_EXPECTS(::stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode), "octex: " + path + " is not a directory");
}

}  // namespace octex_b200
