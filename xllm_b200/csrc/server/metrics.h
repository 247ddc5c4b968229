// Process-wide metrics registry with Prometheus text exposition.
//
// Parity: the bvar-based COUNTER_ADD / GAUGE_SET / HISTOGRAM_OBSERVE families of the reference
// (xllm/core/common/metrics.h:50-120, metrics.cpp) which brpc exports on /vars and /brpc_metrics;
// here the same metric names are served as Prometheus text on /metrics.
#pragma once
#include <algorithm>
#include <map>
#include <mutex>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

namespace xllm {

class Metrics {
 public:
  static Metrics& instance() {
    static Metrics m;
    return m;
  }
  void counter_add(const std::string& name, double v = 1.0) {
    std::lock_guard<std::mutex> lk(mu_);
    counters_[name] += v;
  }
  void gauge_set(const std::string& name, double v) {
    std::lock_guard<std::mutex> lk(mu_);
    gauges_[name] = v;
  }
  void histogram_observe(const std::string& name, double v) {
    std::lock_guard<std::mutex> lk(mu_);
    Hist& h = hists_[name];
    if (h.buckets.empty()) h.buckets.assign(bounds().size() + 1, 0);
    const auto& b = bounds();
    size_t i = std::lower_bound(b.begin(), b.end(), v) - b.begin();
    h.buckets[i]++;
    h.sum += v;
    h.count++;
  }
  double counter(const std::string& name) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = counters_.find(name);
    return it == counters_.end() ? 0.0 : it->second;
  }
  double gauge(const std::string& name) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = gauges_.find(name);
    return it == gauges_.end() ? 0.0 : it->second;
  }
  // Approximate quantile from the bucket counts (upper bound of the bucket that holds it).
  double quantile(const std::string& name, double q) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = hists_.find(name);
    if (it == hists_.end() || it->second.count == 0) return 0.0;
    const double target = q * (double)it->second.count;
    double acc = 0;
    for (size_t i = 0; i < it->second.buckets.size(); ++i) {
      acc += (double)it->second.buckets[i];
      if (acc >= target) return i < bounds().size() ? bounds()[i] : bounds().back() * 2;
    }
    return bounds().back();
  }
  std::string prometheus_text() {
    std::lock_guard<std::mutex> lk(mu_);
    std::string o;
    auto num = [](double v) {
      char buf[48];
      snprintf(buf, sizeof(buf), "%.10g", v);
      return std::string(buf);
    };
    for (auto& kv : counters_) o += "# TYPE " + kv.first + " counter\n" + kv.first + " " + num(kv.second) + "\n";
    for (auto& kv : gauges_) o += "# TYPE " + kv.first + " gauge\n" + kv.first + " " + num(kv.second) + "\n";
    for (auto& kv : hists_) {
      o += "# TYPE " + kv.first + " histogram\n";
      uint64_t acc = 0;
      for (size_t i = 0; i < bounds().size(); ++i) {
        acc += kv.second.buckets[i];
        o += kv.first + "_bucket{le=\"" + num(bounds()[i]) + "\"} " + std::to_string(acc) + "\n";
      }
      o += kv.first + "_bucket{le=\"+Inf\"} " + std::to_string(kv.second.count) + "\n";
      o += kv.first + "_sum " + num(kv.second.sum) + "\n" + kv.first + "_count " + std::to_string(kv.second.count) + "\n";
    }
    return o;
  }
  void reset() {
    std::lock_guard<std::mutex> lk(mu_);
    counters_.clear();
    gauges_.clear();
    hists_.clear();
  }

 private:
  struct Hist {
    std::vector<uint64_t> buckets;
    double sum = 0;
    uint64_t count = 0;
  };
  static const std::vector<double>& bounds() {
    // milliseconds-friendly exponential buckets: 0.1 ms .. ~100 s
    static const std::vector<double> b = [] {
      std::vector<double> v;
      for (double x = 0.1; x < 2e5; x *= 2) v.push_back(x);
      return v;
    }();
    return b;
  }
  std::mutex mu_;
  std::map<std::string, double> counters_, gauges_;
  std::map<std::string, Hist> hists_;
};

}  // namespace xllm
