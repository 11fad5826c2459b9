#include "b200net/param.h"

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstring>

#include "b200net/log.h"

namespace b200net {

std::vector<ParamBase*>& param_registry() {
  static std::vector<ParamBase*> reg;
  return reg;
}

ParamBase::ParamBase(const char* name, const char* doc) : name_(name), doc_(doc ? doc : "") {
  param_registry().push_back(this);
}

ParamBase::~ParamBase() {
  auto& reg = param_registry();
  reg.erase(std::remove(reg.begin(), reg.end(), this), reg.end());
}

const char* ParamBase::find_env(const std::string& name) {
  const std::string own = "B200NET_" + name;
  if (const char* e = getenv(own.c_str())) return e;
  const std::string compat = "OFI_NCCL_" + name;
  return getenv(compat.c_str());
}

void warn_retired(const std::string& name, const char* advice, bool removed) {
  NET_WARN("B200NET_%s / OFI_NCCL_%s is %s. %s", name.c_str(), name.c_str(), removed ? "no longer supported" : "deprecated",
           advice ? advice : "");
}

int parameters_init() {
  int rc = 0;
  for (ParamBase* p : param_registry()) {
    if (p->load_from_env() != 0) {
      NET_WARN("invalid value for parameter %s", p->name().c_str());
      rc = -EINVAL;
    }
  }
  return rc;
}

Params& params() {
  static Params* p = new Params();  // never destroyed: parameters may be read during process teardown
  return *p;
}

static std::string lower(std::string s) {
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
  return s;
}

bool EnumParam::accept(const std::string& v) const {
  const std::string lv = lower(v);
  return std::any_of(allowed_.begin(), allowed_.end(), [&](const std::string& a) { return lower(a) == lv; });
}

namespace detail {

bool parse_value(const char* s, bool& out) {
  const std::string v = lower(s);
  if (v == "1" || v == "true" || v == "yes" || v == "on") { out = true; return true; }
  if (v == "0" || v == "false" || v == "no" || v == "off") { out = false; return true; }
  return false;
}
bool parse_value(const char* s, int64_t& out) {
  if (!*s) return false;
  errno = 0;
  char* end = nullptr;
  const long long v = strtoll(s, &end, 0);
  if (errno || *end) return false;
  out = v;
  return true;
}
bool parse_value(const char* s, uint64_t& out) {
  if (!*s || *s == '-') return false;
  errno = 0;
  char* end = nullptr;
  const unsigned long long v = strtoull(s, &end, 0);
  if (errno || *end) return false;
  out = v;
  return true;
}
bool parse_value(const char* s, int& out) {
  int64_t v;
  if (!parse_value(s, v) || v > INT32_MAX || v < INT32_MIN) return false;
  out = static_cast<int>(v);
  return true;
}
bool parse_value(const char* s, unsigned& out) {
  uint64_t v;
  if (!parse_value(s, v) || v > UINT32_MAX) return false;
  out = static_cast<unsigned>(v);
  return true;
}
bool parse_value(const char* s, float& out) {
  if (!*s) return false;
  errno = 0;
  char* end = nullptr;
  const float v = strtof(s, &end);
  if (errno || *end) return false;
  out = v;
  return true;
}
bool parse_value(const char* s, std::string& out) { out = s; return true; }
std::string to_string_value(bool v) { return v ? "1" : "0"; }
std::string to_string_value(const std::string& v) { return v; }

}  // namespace detail
}  // namespace b200net

// Every parameter with its present value, where the value came from and its description, as a JSON
// array: what `python -m aws_ofi_nccl_b200.utils.params` prints. Returns the length of the whole
// text; at most cap - 1 characters and a terminator are written to out.
extern "C" __attribute__((visibility("default"))) size_t b200net_describe_parameters(char* out, size_t cap) {
  using namespace b200net;
  params();   // the parameter objects register themselves when the set is first built
  auto quoted = [](const std::string& v) {
    std::string q = "\"";
    for (const char c : v) {
      if (c == '"' || c == '\\') q += '\\';
      if (static_cast<unsigned char>(c) >= 0x20) q += c;
    }
    return q + "\"";
  };
  std::string js = "[";
  bool first = true;
  for (ParamBase* p : param_registry()) {
    p->load_from_env();
    const char* src = p->source() == ParamSource::ENVIRONMENT ? "environment" : p->source() == ParamSource::API ? "api" : "default";
    js += std::string(first ? "" : ",") + "{\"name\":" + quoted(p->name()) + ",\"value\":" + quoted(p->value_string()) +
          ",\"source\":\"" + src + "\",\"doc\":" + quoted(p->doc()) + "}";
    first = false;
  }
  js += "]";
  if (out && cap) {
    const size_t n = std::min(js.size(), cap - 1);
    memcpy(out, js.data(), n);
    out[n] = 0;
  }
  return js.size();
}

