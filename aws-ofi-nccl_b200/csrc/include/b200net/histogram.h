// Histogram statistics: histogram<T, Binner> with linear / log2 / custom binners, a timer
// histogram (nanosecond intervals), a scoped timer, and a process-wide registry that prints every
// histogram at finalize in TEXT, TABLE, CSV or JSON form (env OFI_HISTOGRAM_PRINT_FORMAT,
// OFI_HISTOGRAM_SKIP_EMPTY_BINS) (reference: include/stats/*.h, src/stats/histogram.cpp).
#pragma once
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdint>
#include <limits>
#include <mutex>
#include <string>
#include <vector>

namespace b200net::stats {

// A binner maps a value to a bin index in [0, num_bins) and names each bin's lower bound.
template <typename T>
class LinearBinner {
 public:
  LinearBinner(T min, T width, size_t num_bins) : min_(min), width_(width), n_(num_bins) {}
  size_t num_bins() const { return n_; }
  size_t bin_of(T v) const {
    if (v < min_) return 0;
    const size_t b = static_cast<size_t>((v - min_) / width_);
    return b >= n_ ? n_ - 1 : b;
  }
  T lower_bound(size_t bin) const { return min_ + static_cast<T>(bin) * width_; }

 private:
  T min_, width_;
  size_t n_;
};

template <typename T>
class Log2Binner {
 public:
  explicit Log2Binner(size_t num_bins = 40) : n_(num_bins) {}
  size_t num_bins() const { return n_; }
  size_t bin_of(T v) const {
    if (v <= 1) return 0;
    size_t b = 0;
    uint64_t u = static_cast<uint64_t>(v);
    while (u >>= 1) ++b;
    return b >= n_ ? n_ - 1 : b;
  }
  T lower_bound(size_t bin) const { return bin == 0 ? T(0) : static_cast<T>(uint64_t{1} << bin); }

 private:
  size_t n_;
};

// Bin edges given explicitly (ascending); values below the first edge land in bin 0.
template <typename T>
class CustomBinner {
 public:
  explicit CustomBinner(std::vector<T> edges) : edges_(std::move(edges)) {}
  size_t num_bins() const { return edges_.size(); }
  size_t bin_of(T v) const {
    auto it = std::upper_bound(edges_.begin(), edges_.end(), v);
    return it == edges_.begin() ? 0 : static_cast<size_t>(it - edges_.begin()) - 1;
  }
  T lower_bound(size_t bin) const { return edges_[bin]; }

 private:
  std::vector<T> edges_;
};

struct HistogramSnapshot {
  std::string name, unit;
  std::vector<double> lower_bounds;
  std::vector<uint64_t> counts;
  uint64_t samples = 0;
  double min = 0, max = 0, sum = 0;
};

class HistogramBase {
 public:
  virtual ~HistogramBase() = default;
  virtual HistogramSnapshot snapshot() const = 0;
};

void register_histogram(HistogramBase* h);
void unregister_histogram(HistogramBase* h);

template <typename T, typename Binner>
class Histogram : public HistogramBase {
 public:
  Histogram(std::string name, Binner binner, std::string unit = "", bool global = true)
      : name_(std::move(name)), unit_(std::move(unit)), binner_(std::move(binner)), counts_(binner_.num_bins(), 0),
        global_(global) {
    if (global_) register_histogram(this);
  }
  ~Histogram() override {
    if (global_) unregister_histogram(this);
  }
  void insert(T v) {
    std::lock_guard<std::mutex> g(mu_);
    ++counts_[binner_.bin_of(v)];
    ++samples_;
    sum_ += static_cast<double>(v);
    if (samples_ == 1 || v < min_) min_ = v;
    if (samples_ == 1 || v > max_) max_ = v;
  }
  uint64_t samples() const { return samples_; }
  uint64_t count(size_t bin) const { return counts_[bin]; }
  T min() const { return min_; }
  T max() const { return max_; }
  HistogramSnapshot snapshot() const override {
    std::lock_guard<std::mutex> g(mu_);
    HistogramSnapshot s;
    s.name = name_;
    s.unit = unit_;
    s.counts = counts_;
    for (size_t i = 0; i < counts_.size(); ++i) s.lower_bounds.push_back(static_cast<double>(binner_.lower_bound(i)));
    s.samples = samples_;
    s.min = static_cast<double>(min_);
    s.max = static_cast<double>(max_);
    s.sum = sum_;
    return s;
  }

 private:
  std::string name_, unit_;
  Binner binner_;
  std::vector<uint64_t> counts_;
  uint64_t samples_ = 0;
  T min_{}, max_{};
  double sum_ = 0;
  bool global_;
  mutable std::mutex mu_;
};

// Interval histogram in nanoseconds: start()/stop() pairs on one thread.
template <typename Binner = Log2Binner<uint64_t>>
class TimerHistogram : public Histogram<uint64_t, Binner> {
 public:
  explicit TimerHistogram(std::string name, Binner b = Binner(), bool global = true)
      : Histogram<uint64_t, Binner>(std::move(name), std::move(b), "ns", global) {}
  void start() { t0_ = std::chrono::steady_clock::now(); }
  void stop() {
    const auto dt = std::chrono::steady_clock::now() - t0_;
    this->insert(static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(dt).count()));
  }

 private:
  std::chrono::steady_clock::time_point t0_;
};

template <typename TH>
class ScopedTimer {
 public:
  explicit ScopedTimer(TH& h) : h_(h) { h_.start(); }
  ~ScopedTimer() { h_.stop(); }

 private:
  TH& h_;
};

enum class PrintFormat { TEXT, TABLE, CSV, JSON };
PrintFormat print_format_from_env();
std::string format_histogram(const HistogramSnapshot& s, PrintFormat f, bool skip_empty);
// Print every registered histogram (called by the plugin's finalize). Returns how many were printed.
size_t print_all_histograms(FILE* out = nullptr);

}  // namespace b200net::stats
