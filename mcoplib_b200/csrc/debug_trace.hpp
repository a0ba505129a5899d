// Debug aids of the operator shims, controlled at run time by the environment variables mcoplib uses
// (common/mcoplib_ops_params_info.hpp:32-36, common/mcoplib_ops_params_dump.hpp:21-52):
//   MCOP_DEBUG_TRACE=1|ON            print "[MCOP_DEBUG] Call: <operator>" and one line per argument to stdout
//   MCOP_DEBUG_PARAMS_DUMP=<not 0>   write <operator>.json (function, parameters[name, type, dtype, shape, value, bytes])
//   MCOP_TENSOR_DUMP_SAMPLE_SIZE=n   tensor values in the dump: first and last n elements (default 10)
//   MCOP_TENSOR_DUMP_FULL=<not 0>    tensor values in the dump: all elements
// Each variable is read once per process.  With both switches off a call costs two cached boolean tests.
// Dumping values copies the sampled elements to the host and therefore synchronises the stream: debugging only.
#pragma once

#include <ATen/ATen.h>

#include <cstdlib>
#include <fstream>
#include <iostream>
#include <optional>
#include <sstream>
#include <string>
#include <type_traits>
#include <vector>

namespace mcop_debug {

inline bool trace_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("MCOP_DEBUG_TRACE");
    return e != nullptr && (std::string(e) == "1" || std::string(e) == "ON");
  }();
  return on;
}
inline bool dump_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("MCOP_DEBUG_PARAMS_DUMP");
    return e != nullptr && std::string(e) != "0";
  }();
  return on;
}
inline size_t sample_size() {
  static const size_t n = []() -> size_t {
    const char* e = std::getenv("MCOP_TENSOR_DUMP_SAMPLE_SIZE");
    if (!e) return 10;
    char* end = nullptr;
    const unsigned long v = std::strtoul(e, &end, 10);
    return (end != e && v > 0) ? (size_t)v : 10;
  }();
  return n;
}
inline bool dump_full() {
  static const bool on = [] {
    const char* e = std::getenv("MCOP_TENSOR_DUMP_FULL");
    return e != nullptr && std::string(e) != "0";
  }();
  return on;
}

struct Param {
  std::string name, type, dtype, shape, value;
  size_t bytes = 0;
};

template <typename T> struct is_optional : std::false_type {};
template <typename T> struct is_optional<std::optional<T>> : std::true_type {};

template <typename T> inline const char* scalar_name() {
  if (std::is_same<T, bool>::value) return "bool";
  if (std::is_same<T, int>::value) return "int";
  if (std::is_same<T, long>::value || std::is_same<T, long long>::value) return "long";
  if (std::is_same<T, float>::value) return "float";
  if (std::is_same<T, double>::value) return "double";
  return "scalar";
}

inline std::string shape_string(const at::Tensor& t) {
  std::ostringstream ss;
  ss << "[";
  for (int64_t i = 0; i < t.dim(); ++i) ss << (i ? ", " : "") << t.size(i);
  ss << "]";
  return ss.str();
}

// the line of the trace: Tensor(Shape=[a, b], Dtype=BFloat16, Device=cuda:0)
inline void print_value(std::ostream& os, const at::Tensor& t) {
  if (!t.defined()) { os << "Tensor(Undefined)"; return; }
  os << "Tensor(Shape=" << shape_string(t) << ", Dtype=" << t.scalar_type() << ", Device=" << t.device() << ")";
}
template <typename T> inline void print_value(std::ostream& os, const T& v) { os << v; }
template <typename T> inline void print_value(std::ostream& os, const std::optional<T>& v) {
  if (v.has_value()) { os << "Optional("; print_value(os, *v); os << ")"; } else os << "Optional(nullopt)";
}

inline std::string tensor_values(const at::Tensor& t) {
  const int64_t total = t.numel();
  const int64_t n = (int64_t)sample_size();
  std::ostringstream ss;
  const bool integral = at::isIntegralType(t.scalar_type(), /*includeBool=*/true);
  auto emit = [&](const at::Tensor& part) {
    if (integral) {
      const at::Tensor h = part.to(at::kCPU).to(at::kLong).contiguous();
      const int64_t* d = h.data_ptr<int64_t>();
      for (int64_t i = 0; i < h.numel(); ++i) ss << (i ? ", " : "") << d[i];
    } else {
      const at::Tensor h = part.to(at::kCPU).to(at::kDouble).contiguous();
      const double* d = h.data_ptr<double>();
      for (int64_t i = 0; i < h.numel(); ++i) ss << (i ? ", " : "") << d[i];
    }
  };
  ss << "[";
  if (total > 0) {
    const at::Tensor flat = t.reshape({-1});
    if (dump_full() || total <= 2 * n) {
      emit(flat);
    } else {
      emit(flat.slice(0, 0, n));
      ss << ", ..., ";
      emit(flat.slice(0, total - n, total));
    }
  }
  ss << "]";
  return ss.str();
}

inline Param describe(const at::Tensor& t) {
  Param p;
  p.type = "at::Tensor";
  if (!t.defined()) { p.dtype = "undefined"; p.shape = "[]"; p.value = "undefined"; return p; }
  std::ostringstream dt;
  dt << t.scalar_type();
  p.dtype = dt.str();
  p.shape = shape_string(t);
  p.bytes = (size_t)t.numel() * t.element_size();
  try { p.value = tensor_values(t); } catch (const std::exception&) { p.value = "[... (values unavailable)]"; }
  return p;
}
template <typename T> inline Param describe(const T& v) {
  Param p;
  p.type = p.dtype = scalar_name<T>();
  p.shape = "[]";
  std::ostringstream ss;
  ss << v;
  p.value = ss.str();
  p.bytes = sizeof(T);
  return p;
}
template <typename T> inline Param describe(const std::optional<T>& v) {
  if (!v.has_value()) {
    Param p;
    p.type = "std::optional"; p.dtype = "nullopt"; p.shape = "[]"; p.value = "nullopt";
    return p;
  }
  Param p = describe(*v);
  p.type = "std::optional<" + p.type + ">";
  return p;
}

inline std::string escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (c == '\n') o += "\\n";
    else o += c;
  }
  return o;
}

// "a, b, c" (the stringified argument list of the macro below) -> {"a", "b", "c"}
inline std::vector<std::string> split_names(const char* s) {
  std::vector<std::string> out;
  std::string cur;
  int depth = 0;
  for (const char* c = s; *c; ++c) {
    if (*c == '(' || *c == '<' || *c == '[') ++depth;
    if (*c == ')' || *c == '>' || *c == ']') --depth;
    if (*c == ',' && depth == 0) { out.push_back(cur); cur.clear(); continue; }
    if (*c == ' ' && cur.empty()) continue;
    cur += *c;
  }
  if (!cur.empty()) out.push_back(cur);
  return out;
}

template <typename... Args>
inline void call(const char* op, const char* names_csv, const Args&... args) {
  const bool tr = trace_enabled(), du = dump_enabled();
  if (!tr && !du) return;
  const std::vector<std::string> names = split_names(names_csv);
  if (tr) {
    std::cout << "[MCOP_DEBUG] Call: " << op << "\n";
    size_t i = 0;
    const size_t n = sizeof...(Args);
    (void)std::initializer_list<int>{(std::cout << "  " << (i < names.size() ? names[i] : std::string("arg")) << " = ",
                                       print_value(std::cout, args), std::cout << (++i < n ? ",\n" : ""), 0)...};
    std::cout << std::endl;
  }
  if (du) {
    try {
      std::vector<Param> params{describe(args)...};
      std::ostringstream ss;
      ss << "{\n  \"function\": \"" << escape(op) << "\",\n  \"parameters\": [\n";
      for (size_t i = 0; i < params.size(); ++i) {
        const Param& p = params[i];
        ss << "    {\n      \"name\": \"" << escape(i < names.size() ? names[i] : "arg" + std::to_string(i)) << "\",\n"
           << "      \"type\": \"" << escape(p.type) << "\",\n      \"dtype\": \"" << escape(p.dtype) << "\",\n"
           << "      \"shape\": \"" << escape(p.shape) << "\",\n      \"value\": \"" << escape(p.value) << "\",\n"
           << "      \"bytes\": " << p.bytes << "\n    }" << (i + 1 < params.size() ? "," : "") << "\n";
      }
      ss << "  ]\n}\n";
      std::ofstream f(std::string(op) + ".json", std::ios::out | std::ios::trunc);
      if (f.is_open()) f << ss.str();
    } catch (const std::exception&) {
      // a failed dump never disturbs the operator
    }
  }
}

}  // namespace mcop_debug

// First statement of every operator shim: MCOP_DEBUG_CALL("operator_name", arg1, arg2, ...)
#define MCOP_DEBUG_CALL(op, ...) ::mcop_debug::call(op, #__VA_ARGS__, __VA_ARGS__)
