// Stand-in for spdlog: logging calls of the reference compile to nothing.
#pragma once
namespace spdlog {
template <typename... Args> void debug(const char *, Args &&...) {}
template <typename... Args> void info(const char *, Args &&...) {}
template <typename... Args> void warn(const char *, Args &&...) {}
template <typename... Args> void error(const char *, Args &&...) {}
template <typename... Args> void critical(const char *, Args &&...) {}
} // namespace spdlog
