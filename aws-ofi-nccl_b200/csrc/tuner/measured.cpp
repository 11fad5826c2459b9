#include <cctype>
#include <cmath>
#include <cstdlib>
#include <limits>
#include <map>
#include <cstdio>

#include "b200net/log.h"
#include "b200net/tuner/tuner.h"

namespace b200net::tuner {

// Minimal reader for the calibration file: finds "key": number pairs inside each {...} of "rows".
static bool parse_number_after(const std::string& s, size_t from, size_t to, const char* key, double* out) {
  const std::string k = std::string("\"") + key + "\"";
  const size_t p = s.find(k, from);
  if (p == std::string::npos || p >= to) return false;
  size_t c = s.find(':', p + k.size());
  if (c == std::string::npos || c >= to) return false;
  ++c;
  while (c < to && std::isspace(static_cast<unsigned char>(s[c]))) ++c;
  char* end = nullptr;
  const double v = strtod(s.c_str() + c, &end);
  if (end == s.c_str() + c) return false;
  *out = v;
  return true;
}

bool MeasuredTuner::load_from_string(const std::string& json) {
  rows_.clear();
  world_ = 0;
  const size_t rows_at = json.find("\"rows\"");
  if (rows_at == std::string::npos) return false;
  double w = 0;
  if (parse_number_after(json, 0, rows_at, "world", &w)) world_ = static_cast<size_t>(w);
  size_t pos = json.find('[', rows_at);
  if (pos == std::string::npos) return false;
  for (;;) {
    const size_t open = json.find('{', pos);
    const size_t close_arr = json.find(']', pos);
    if (open == std::string::npos || (close_arr != std::string::npos && close_arr < open)) break;
    const size_t close = json.find('}', open);
    if (close == std::string::npos) return false;
    double coll, algo, proto, nch = 0, bytes, t;
    if (!parse_number_after(json, open, close, "coll", &coll) || !parse_number_after(json, open, close, "algo", &algo) ||
        !parse_number_after(json, open, close, "proto", &proto) || !parse_number_after(json, open, close, "bytes", &bytes) ||
        !parse_number_after(json, open, close, "time_us", &t)) {
      rows_.clear();
      return false;
    }
    parse_number_after(json, open, close, "nchannels", &nch);
    if (t > 0 && coll >= 0 && coll < ncclNumFuncs && algo >= 0 && algo < NCCL_NUM_ALGORITHMS && proto >= 0 &&
        proto < NCCL_NUM_PROTOCOLS)
      rows_.push_back(MeasuredRow{static_cast<int>(coll), static_cast<int>(algo), static_cast<int>(proto),
                                  static_cast<int>(nch), static_cast<size_t>(bytes), t});
    pos = close + 1;
  }
  return !rows_.empty();
}

bool MeasuredTuner::load(const std::string& path) {
  FILE* f = fopen(path.c_str(), "r");
  if (!f) return false;
  std::string text;
  char buf[4096];
  size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
  fclose(f);
  const bool ok = load_from_string(text);
  if (!ok) NET_WARN("tuner table %s is malformed or empty", path.c_str());
  return ok;
}

Decision MeasuredTuner::decide(ncclFunc_t coll, size_t bytes) const {
  Decision d;
  if (rows_.empty() || bytes == 0) return d;
  // nearest measured size on a log scale, then the fastest row at that size
  double best_dist = std::numeric_limits<double>::max();
  size_t nearest = 0;
  bool any = false;
  const double lb = std::log2(static_cast<double>(bytes));
  for (const MeasuredRow& r : rows_) {
    if (r.coll != static_cast<int>(coll)) continue;
    const double dist = std::fabs(std::log2(static_cast<double>(r.bytes)) - lb);
    if (dist < best_dist) {
      best_dist = dist;
      nearest = r.bytes;
      any = true;
    }
  }
  if (!any) return d;
  double best_t = std::numeric_limits<double>::max();
  for (const MeasuredRow& r : rows_) {
    if (r.coll != static_cast<int>(coll) || r.bytes != nearest) continue;
    if (r.time_us < best_t) {
      best_t = r.time_us;
      d.algorithm = r.algo;
      d.protocol = r.proto;
      d.n_channels = r.n_channels;
    }
  }
  return d;
}

}  // namespace b200net::tuner
