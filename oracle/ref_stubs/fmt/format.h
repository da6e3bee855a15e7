// Stand-in for {fmt}: format() is named by templates of the reference's util.h that are never
// instantiated here.
#pragma once
#include <string>
namespace fmt {
template <typename... Args> std::string format(const char *f, Args &&...) { return std::string(f); }
} // namespace fmt
