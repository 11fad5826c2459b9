#include <algorithm>
#include <cctype>
#include <vector>
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
    double reg = -1;
    parse_number_after(json, open, close, "reg", &reg);
    // algo / proto -1: the row times a channel count with the algorithm and protocol left to NCCL
    // (sweeps of the transport's channel count); such a row decides channels only
    const bool nccl_choice = algo < 0 && proto < 0;
    if (t > 0 && coll >= 0 && coll < ncclNumFuncs &&
        (nccl_choice || (algo >= 0 && algo < NCCL_NUM_ALGORITHMS && proto >= 0 && proto < NCCL_NUM_PROTOCOLS)))
      rows_.push_back(MeasuredRow{static_cast<int>(coll), nccl_choice ? NCCL_ALGO_UNDEF : static_cast<int>(algo),
                                  nccl_choice ? NCCL_PROTO_UNDEF : static_cast<int>(proto),
                                  static_cast<int>(nch), static_cast<size_t>(bytes), t, reg < 0 ? -1 : (reg != 0 ? 1 : 0)});
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

Decision MeasuredTuner::decide(ncclFunc_t coll, size_t bytes, int reg_buff) const {
  Decision d;
  if (rows_.empty() || bytes == 0) return d;
  // rows of this collective; when the caller says whether its buffers are registered and the
  // table recorded that for this collective, only rows of the same kind
  bool table_knows_reg = false;
  for (const MeasuredRow& r : rows_)
    if (r.coll == static_cast<int>(coll) && r.reg >= 0) table_knows_reg = true;
  auto usable = [&](const MeasuredRow& r) {
    if (r.coll != static_cast<int>(coll)) return false;
    return !(reg_buff >= 0 && table_knows_reg && r.reg >= 0 && r.reg != (reg_buff ? 1 : 0));
  };
  // the measured sizes that bracket the request
  size_t below = 0, above = 0;
  for (const MeasuredRow& r : rows_) {
    if (!usable(r)) continue;
    if (r.bytes <= bytes && r.bytes > below) below = r.bytes;
    if (r.bytes >= bytes && (above == 0 || r.bytes < above)) above = r.bytes;
  }
  if (below == 0 && above == 0) return d;
  if (below == 0) below = above;
  if (above == 0) above = below;
  // estimated time per (algorithm, protocol); at each bracketing size the combination's best row
  // counts, rows within 3 % of it tie and the one with the fewest channels stands for it
  struct Cand { int algo, proto; double t_lo, t_hi; int nch_lo, nch_hi; };
  std::vector<Cand> cands;
  auto cand_of = [&](const MeasuredRow& r) -> Cand& {
    for (Cand& c : cands)
      if (c.algo == r.algo && c.proto == r.proto) return c;
    cands.push_back(Cand{r.algo, r.proto, -1.0, -1.0, 0, 0});
    return cands.back();
  };
  auto better = [](double t, int nch, double cur_t, int cur_nch) {
    if (cur_t < 0) return true;
    if (t < cur_t / 1.03) return true;                       // clearly faster
    if (t <= cur_t * 1.03 && nch < cur_nch) return true;     // tied: fewer channels
    return false;
  };
  for (const MeasuredRow& r : rows_) {
    if (!usable(r)) continue;
    if (r.bytes == below) {
      Cand& c = cand_of(r);
      if (better(r.time_us, r.n_channels, c.t_lo, c.nch_lo)) { c.t_lo = r.time_us; c.nch_lo = r.n_channels; }
    }
    if (r.bytes == above) {
      Cand& c = cand_of(r);
      if (better(r.time_us, r.n_channels, c.t_hi, c.nch_hi)) { c.t_hi = r.time_us; c.nch_hi = r.n_channels; }
    }
  }
  const double w = above == below ? 0.0
                                  : (std::log2(static_cast<double>(bytes)) - std::log2(static_cast<double>(below))) /
                                        (std::log2(static_cast<double>(above)) - std::log2(static_cast<double>(below)));
  const bool near_lo = w < 0.5;
  // a combination measured on one side only stands with that side's time when that side is the
  // nearer one; measured on the far side only it is no candidate (its time there says little here)
  auto estimate = [&](const Cand& c) {
    if (c.t_lo >= 0 && c.t_hi >= 0) return std::exp2((1.0 - w) * std::log2(c.t_lo) + w * std::log2(c.t_hi));
    if (c.t_lo >= 0) return near_lo ? c.t_lo : -1.0;
    return near_lo ? -1.0 : c.t_hi;
  };
  auto channels = [&](const Cand& c) { return (near_lo && c.t_lo >= 0) || c.t_hi < 0 ? c.nch_lo : c.nch_hi; };
  double best = std::numeric_limits<double>::max();
  for (const Cand& c : cands)
    if (estimate(c) >= 0) best = std::min(best, estimate(c));
  const Cand* pick = nullptr;
  for (const Cand& c : cands) {
    const double e = estimate(c);
    if (e < 0 || e > best * 1.03) continue;
    if (!pick || channels(c) < channels(*pick) || (channels(c) == channels(*pick) && e < estimate(*pick))) pick = &c;
  }
  if (!pick) {
    // everything was measured on the far side only: let that side decide
    for (const Cand& c : cands) {
      const double e = c.t_lo >= 0 ? c.t_lo : c.t_hi;
      if (!pick || e < (pick->t_lo >= 0 ? pick->t_lo : pick->t_hi)) pick = &c;
    }
    if (!pick) return d;
  }
  d.algorithm = pick->algo;
  d.protocol = pick->proto;
  d.n_channels = channels(*pick);
  return d;
}

}  // namespace b200net::tuner
