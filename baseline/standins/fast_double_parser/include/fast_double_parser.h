// Stand-in for the fast_double_parser header-only library, used only to build the
// reference framework offline for benchmarking (its external_libs submodules are
// empty in the mounted tree). One entry point is needed: parse_number(p, out)
// returns the end of the parsed number, or nullptr when nothing could be parsed so
// that the caller falls back to its own strtod path. Text parsing is never on a
// timed path of the benchmark (data is passed as in-memory matrices).
#ifndef FAST_DOUBLE_PARSER_STANDIN_H_
#define FAST_DOUBLE_PARSER_STANDIN_H_

#include <cstdlib>

namespace fast_double_parser {

inline const char* parse_number(const char* p, double* out) {
  // the real library accepts only JSON-style numbers: [-]digits[.digits][e[+-]digits]
  const char* q = p;
  if (*q == '-') ++q;
  if (!(*q >= '0' && *q <= '9')) return nullptr;
  char* end = nullptr;
  double v = std::strtod(p, &end);
  if (end == p) return nullptr;
  *out = v;
  return end;
}

}  // namespace fast_double_parser

#endif  // FAST_DOUBLE_PARSER_STANDIN_H_
