// Minimal stand-in for llvm/Support/raw_ostream.h, used only to compile the
// reference's arithmetic sources outside an LLVM tree (test infrastructure).
#pragma once
#include <cstdio>
#include <cstdlib>
#include <string>
namespace llvm {
class raw_ostream {
public:
  raw_ostream &operator<<(const char *s) { std::fputs(s, stderr); return *this; }
  raw_ostream &operator<<(const std::string &s) { std::fputs(s.c_str(), stderr); return *this; }
  raw_ostream &operator<<(char c) { std::fputc(c, stderr); return *this; }
  raw_ostream &operator<<(long long v) { std::fprintf(stderr, "%lld", v); return *this; }
  raw_ostream &operator<<(unsigned long long v) { std::fprintf(stderr, "%llu", v); return *this; }
  raw_ostream &operator<<(long v) { std::fprintf(stderr, "%ld", v); return *this; }
  raw_ostream &operator<<(unsigned long v) { std::fprintf(stderr, "%lu", v); return *this; }
  raw_ostream &operator<<(int v) { std::fprintf(stderr, "%d", v); return *this; }
  raw_ostream &operator<<(unsigned v) { std::fprintf(stderr, "%u", v); return *this; }
  raw_ostream &operator<<(double v) { std::fprintf(stderr, "%g", v); return *this; }
};
inline raw_ostream &errs() { static raw_ostream s; return s; }
inline raw_ostream &outs() { static raw_ostream s; return s; }
inline raw_ostream &dbgs() { static raw_ostream s; return s; }
} // namespace llvm
#ifndef llvm_unreachable
#define llvm_unreachable(msg) do { std::fprintf(stderr, "unreachable: %s\n", msg); std::abort(); } while (0)
#endif
