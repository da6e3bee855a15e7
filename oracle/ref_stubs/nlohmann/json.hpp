// Stand-in for nlohmann::json: the interface one helper of the reference's util.cpp uses.
#pragma once
#include <string>
namespace nlohmann {
class json {
public:
  bool contains(const char *) const { return false; }
  const json &operator[](const char *) const { return *this; }
  bool is_object() const { return false; }
  std::string value(const char *, const char *fallback) const { return fallback; }
};
} // namespace nlohmann
