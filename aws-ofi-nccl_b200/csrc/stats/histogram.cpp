#include "b200net/histogram.h"

#include <cstdlib>
#include <cstring>
#include <cmath>
#include <cstdio>

namespace b200net::stats {

static std::mutex& reg_mu() {
  static std::mutex m;
  return m;
}
static std::vector<HistogramBase*>& reg() {
  static std::vector<HistogramBase*> r;
  return r;
}

void register_histogram(HistogramBase* h) {
  std::lock_guard<std::mutex> g(reg_mu());
  reg().push_back(h);
}
void unregister_histogram(HistogramBase* h) {
  std::lock_guard<std::mutex> g(reg_mu());
  auto& r = reg();
  r.erase(std::remove(r.begin(), r.end(), h), r.end());
}

PrintFormat print_format_from_env() {
  const char* e = getenv("OFI_HISTOGRAM_PRINT_FORMAT");
  if (!e) return PrintFormat::TEXT;
  if (!strcasecmp(e, "TABLE")) return PrintFormat::TABLE;
  if (!strcasecmp(e, "CSV")) return PrintFormat::CSV;
  if (!strcasecmp(e, "JSON")) return PrintFormat::JSON;
  return PrintFormat::TEXT;
}

static std::string num(double v) {
  char b[64];
  if (v == static_cast<double>(static_cast<long long>(v)) && std::fabs(v) < 1e15)
    snprintf(b, sizeof(b), "%lld", static_cast<long long>(v));
  else
    snprintf(b, sizeof(b), "%g", v);
  return b;
}

std::string format_histogram(const HistogramSnapshot& s, PrintFormat f, bool skip_empty) {
  std::string o;
  const double mean = s.samples ? s.sum / static_cast<double>(s.samples) : 0.0;
  const std::string samples = std::to_string(s.samples);
  switch (f) {
    case PrintFormat::TEXT:
      o += "histogram " + s.name + " (" + s.unit + "): samples=" + samples + " min=" + num(s.min) + " max=" + num(s.max) +
           " mean=" + num(mean) + "\n";
      for (size_t i = 0; i < s.counts.size(); ++i) {
        if (skip_empty && !s.counts[i]) continue;
        o += "  >= " + num(s.lower_bounds[i]) + " : " + std::to_string(s.counts[i]) + "\n";
      }
      break;
    case PrintFormat::TABLE:
      o += "| " + s.name + " | lower bound (" + s.unit + ") | count |\n|---|---|---|\n";
      for (size_t i = 0; i < s.counts.size(); ++i) {
        if (skip_empty && !s.counts[i]) continue;
        o += "| | " + num(s.lower_bounds[i]) + " | " + std::to_string(s.counts[i]) + " |\n";
      }
      o += "| total | | " + samples + " |\n";
      break;
    case PrintFormat::CSV:
      o += "name,unit,lower_bound,count\n";
      for (size_t i = 0; i < s.counts.size(); ++i) {
        if (skip_empty && !s.counts[i]) continue;
        o += s.name + "," + s.unit + "," + num(s.lower_bounds[i]) + "," + std::to_string(s.counts[i]) + "\n";
      }
      break;
    case PrintFormat::JSON: {
      o += "{\"name\":\"" + s.name + "\",\"unit\":\"" + s.unit + "\",\"samples\":" + samples + ",\"min\":" + num(s.min) +
           ",\"max\":" + num(s.max) + ",\"mean\":" + num(mean) + ",\"bins\":[";
      bool first = true;
      for (size_t i = 0; i < s.counts.size(); ++i) {
        if (skip_empty && !s.counts[i]) continue;
        if (!first) o += ",";
        first = false;
        o += "{\"ge\":" + num(s.lower_bounds[i]) + ",\"count\":" + std::to_string(s.counts[i]) + "}";
      }
      o += "]}\n";
      break;
    }
  }
  return o;
}

size_t print_all_histograms(FILE* out) {
  if (!out) out = stderr;
  const PrintFormat f = print_format_from_env();
  const char* se = getenv("OFI_HISTOGRAM_SKIP_EMPTY_BINS");
  const bool skip = !se || strcmp(se, "0") != 0;
  std::vector<HistogramSnapshot> snaps;
  {
    std::lock_guard<std::mutex> g(reg_mu());
    for (HistogramBase* h : reg()) snaps.push_back(h->snapshot());
  }
  size_t n = 0;
  for (const auto& s : snaps) {
    if (!s.samples) continue;
    fputs(format_histogram(s, f, skip).c_str(), out);
    ++n;
  }
  return n;
}

}  // namespace b200net::stats
